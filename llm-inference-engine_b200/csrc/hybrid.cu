// hybrid.cu -- the layer-list decoder: a model given as a list of layers, each with a token mixer of some kind and an optional
// feed-forward of some kind (b200_hybrid_layer_t), run over a ragged mixed batch of portions (b200_hybrid_batch_t).
//
// One layer = x += rmsnorm(mixer(x)) * g1;  x += rmsnorm(ff(x)) * g2, with x the fp32 residual stream.  Launch sequence per layer:
//   fused input projection (b200_linear: tcgen05 GEMM / weight-streaming GEMV by token count)
//   attention mixer:  q/k whole-projection norm + pool append -> chunked sink attention (gate fused) -> output projection
//   gla mixer:        decay (low-rank, fp32) -> recurrence over the state slots -> head norm * silu(gate) -> output projection
//   post-norm + residual add (fp32)
//   moe:              router + shared gate (fp32) -> route -> plan -> gather (weight on the input) -> grouped up (+act) -> grouped down
//                     shared expert: b200_linear up -> act -> b200_linear down
//                     combine (sum of the token's expert rows + gate * shared) + post-norm + residual add, one kernel
// and at the end: final norm of the wanted rows -> LM head with fp32 logits.
// Everything is stream-ordered and allocation-free; the only host->device traffic of a call is one copy of the batch description.
#include "hybrid_ops.cuh"

#include <new>
#include <vector>

namespace b200 {

constexpr int kPageH = B200_KV_PAGE_SIZE;
static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <typename T>
__global__ void embed_f32_kernel(const int *__restrict__ ids, const T *__restrict__ table, float *__restrict__ x, T *__restrict__ h, int width,
                                 int vocab) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host has refused ids outside the vocabulary
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const T v = table[(size_t)id * width + c];
        x[(size_t)t * width + c] = Elem<T>::to_f(v);
        if (h) h[(size_t)t * width + c] = v;  // the 16-bit copy the first projection reads
    }
}

// x[t, :] += rmsnorm(y[t, :]) * g (and h_out[t, :] = T(x[t, :]) for the next projection), where y is either a dense row (y_dense) or the mixture
//   sum_k y_rows[pair_row[t*top + k], :] + shared_gate[t] * y_shared[t, :].   trace (optional) receives the new x.
template <typename T>
__global__ void __launch_bounds__(256)
postnorm_residual_kernel(float *__restrict__ x, const T *__restrict__ y_dense, const T *__restrict__ y_rows, const int *__restrict__ pair_row,
                         int top, const T *__restrict__ y_shared, const float *__restrict__ shared_gate, const float *__restrict__ g, float eps,
                         int width, float *__restrict__ trace, T *__restrict__ h_out) {
    extern __shared__ __align__(16) float ys[];  // [width]
    __shared__ float red[33];
    const int t = blockIdx.x;
    constexpr int V = Elem<T>::kVec;
    // 16-byte pieces when every row starts on a 16-byte boundary (the sums are formed in the same order as element by element)
    const bool vec = width % V == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(y_dense) | reinterpret_cast<size_t>(y_rows) |
                                         reinterpret_cast<size_t>(y_shared) | reinterpret_cast<size_t>(g) | reinterpret_cast<size_t>(trace) |
                                         reinterpret_cast<size_t>(h_out)) & 15) == 0;
    float ss = 0.0f;
    if (vec) {
        const float sg = (!y_dense && y_shared) ? shared_gate[t] : 0.0f;
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
            float v[V];
            if (y_dense) {
                unpack16<T>(ld_v4(y_dense + (size_t)t * width + c), v);
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) v[i] = 0.0f;
                for (int k = 0; k < top; ++k) {
                    float f[V];
                    unpack16<T>(ld_v4(y_rows + (size_t)pair_row[(size_t)t * top + k] * width + c), f);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] += f[i];
                }
                if (y_shared) {
                    float f[V];
                    unpack16<T>(ld_v4(y_shared + (size_t)t * width + c), f);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] = fmaf(sg, f[i], v[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < V; i += 4) *reinterpret_cast<float4 *>(ys + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
            for (int i = 0; i < V; ++i) ss = fmaf(v[i], v[i], ss);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float v;
            if (y_dense) {
                v = Elem<T>::to_f(y_dense[(size_t)t * width + c]);
            } else {
                v = 0.0f;
                for (int k = 0; k < top; ++k) v += Elem<T>::to_f(y_rows[(size_t)pair_row[(size_t)t * top + k] * width + c]);
                if (y_shared) v = fmaf(shared_gate[t], Elem<T>::to_f(y_shared[(size_t)t * width + c]), v);
            }
            ys[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    if (vec) {
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {  // a thread reads back the pieces of ys it wrote
            float v[V];
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 xv = *reinterpret_cast<const float4 *>(x + (size_t)t * width + c + i);
                const float4 gv = *reinterpret_cast<const float4 *>(g + c + i);
                const float4 yv = *reinterpret_cast<const float4 *>(ys + c + i);
                const float4 r = make_float4(xv.x + yv.x * inv * gv.x, xv.y + yv.y * inv * gv.y, xv.z + yv.z * inv * gv.z, xv.w + yv.w * inv * gv.w);
                *reinterpret_cast<float4 *>(x + (size_t)t * width + c + i) = r;
                if (trace) *reinterpret_cast<float4 *>(trace + (size_t)t * width + c + i) = r;
                v[i] = r.x, v[i + 1] = r.y, v[i + 2] = r.z, v[i + 3] = r.w;
            }
            if (h_out) st_v4(h_out + (size_t)t * width + c, pack16<T>(v));  // what the next sublayer's projections read (16-bit engines)
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[(size_t)t * width + c] + ys[c] * inv * g[c];
        x[(size_t)t * width + c] = v;
        if (trace) trace[(size_t)t * width + c] = v;
        if (h_out) h_out[(size_t)t * width + c] = Elem<T>::from_f(v);  // what the next sublayer's projections read (16-bit engines)
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
final_norm_rows_kernel(const float *__restrict__ x, const int *__restrict__ rows, const float *__restrict__ g, float eps, float *__restrict__ out,
                       T *__restrict__ out_t, int width) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    const float *xr = x + (size_t)rows[i] * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = xr[c] * inv * g[c];
        out[(size_t)i * width + c] = v;
        if (out_t) out_t[(size_t)i * width + c] = Elem<T>::from_f(v);
    }
}

// y[m, n] = sum_k x[m, k] w[n, k] (+ bias[n]), fp32 out: used where the result must stay fp32 (router logits, the LM head).
// A CTA stages PM rows of x in shared memory (fp32) and its 8 warps walk the CTA's slice of output columns: a weight row is read once per
// PM activations and the activations once per CTA.
template <typename TX, typename TW, int PM>
__global__ void __launch_bounds__(256)
proj_f32_kernel(const TX *__restrict__ x, int ldx, const TW *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y, int ldy, int M,
                int N, int K, int cols_per_cta) {
    extern __shared__ float xs[];  // [PM][K]
    const int m0 = blockIdx.y * PM, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < PM * K; i += blockDim.x) {
        const int mm = i / K, k = i - mm * K;
        xs[i] = m0 + mm < M ? Elem<TX>::to_f(x[(size_t)(m0 + mm) * ldx + k]) : 0.0f;
    }
    __syncthreads();
    const int n_end = min(N, (int)(blockIdx.x + 1) * cols_per_cta);
    for (int n = blockIdx.x * cols_per_cta + warp; n < n_end; n += 8) {
        float acc[PM] = {};
        const TW *wr = w + (size_t)n * K;
        for (int k = lane; k < K; k += 32) {
            const float wv = Elem<TW>::to_f(wr[k]);
#pragma unroll
            for (int i = 0; i < PM; ++i) acc[i] = fmaf(xs[i * K + k], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < PM; ++i) {
            const float v = warp_sum(acc[i]);
            if (lane == 0 && m0 + i < M) y[(size_t)(m0 + i) * ldy + n] = v + (bias ? bias[n] : 0.0f);
        }
    }
}

// Few outputs (a decode batch's router logits): one warp per output element, four independent partial sums per lane.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
proj_f32_small_kernel(const TX *__restrict__ x, int ldx, const TW *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y, int ldy,
                      int M, int N, int K) {
    const int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (o >= M * N) return;
    const int mrow = o / N, n = o - mrow * N;
    const TX *xr = x + (size_t)mrow * ldx;
    const TW *wr = w + (size_t)n * K;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    int k = lane;
    for (; k + 96 < K; k += 128) {
        a0 = fmaf(Elem<TX>::to_f(xr[k]), Elem<TW>::to_f(wr[k]), a0);
        a1 = fmaf(Elem<TX>::to_f(xr[k + 32]), Elem<TW>::to_f(wr[k + 32]), a1);
        a2 = fmaf(Elem<TX>::to_f(xr[k + 64]), Elem<TW>::to_f(wr[k + 64]), a2);
        a3 = fmaf(Elem<TX>::to_f(xr[k + 96]), Elem<TW>::to_f(wr[k + 96]), a3);
    }
    for (; k < K; k += 32) a0 = fmaf(Elem<TX>::to_f(xr[k]), Elem<TW>::to_f(wr[k]), a0);
    const float v = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) y[(size_t)mrow * ldy + n] = v + (bias ? bias[n] : 0.0f);
}

template <typename TX, typename TW, int PM>
static void launch_proj_f32_t(const void *x, int ldx, const void *w, const float *bias, float *y, int ldy, int M, int N, int K, cudaStream_t st) {
    const size_t smem = (size_t)PM * K * sizeof(float);
    // enough CTAs to fill the device, at least 8 columns (one per warp) each
    const int mt = (M + PM - 1) / PM;
    int cols = (N * mt + 4 * 148 - 1) / (4 * 148);
    cols = cols < 8 ? 8 : (cols + 7) / 8 * 8;
    if (smem > 48 * 1024) cudaFuncSetAttribute(proj_f32_kernel<TX, TW, PM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    proj_f32_kernel<TX, TW, PM><<<dim3((N + cols - 1) / cols, mt), 256, smem, st>>>((const TX *)x, ldx, (const TW *)w, bias, y, ldy, M, N, K, cols);
}

int launch_proj_f32(int x_dtype, const void *x, int ldx, int w_dtype, const void *w, const float *bias, float *y, int ldy, int M, int N,
                    int K, cudaStream_t st) {
    if (M == 0) return B200_OK;
    if ((long long)M * N <= 8192) {
        const int grid = (M * N + 7) / 8;
        B200_DISPATCH_DTYPE(w_dtype, {
            if (x_dtype == B200_F32) proj_f32_small_kernel<float, T><<<grid, 256, 0, st>>>((const float *)x, ldx, (const T *)w, bias, y, ldy, M, N, K);
            else proj_f32_small_kernel<T, T><<<grid, 256, 0, st>>>((const T *)x, ldx, (const T *)w, bias, y, ldy, M, N, K);
        });
        return cuda_status("proj_f32 (small) launch");
    }
    if ((size_t)4 * K * sizeof(float) > 200 * 1024) {
        set_error("proj_f32: K = %d does not fit the shared-memory activation tile", K);
        return B200_ERR_UNSUPPORTED;
    }
    const bool wide = M > 8 && (size_t)16 * K * sizeof(float) <= 200 * 1024, mid = (size_t)8 * K * sizeof(float) <= 200 * 1024;
    B200_DISPATCH_DTYPE(w_dtype, {
        if (x_dtype == B200_F32) {
            if (wide) launch_proj_f32_t<float, T, 16>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else if (mid) launch_proj_f32_t<float, T, 8>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else launch_proj_f32_t<float, T, 4>(x, ldx, w, bias, y, ldy, M, N, K, st);
        } else {
            if (wide) launch_proj_f32_t<T, T, 16>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else if (mid) launch_proj_f32_t<T, T, 8>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else launch_proj_f32_t<T, T, 4>(x, ldx, w, bias, y, ldy, M, N, K, st);
        }
    });
    return cuda_status("proj_f32 launch");
}

struct LayerPlan {
    int n_in = 0;                     // rows of the fused input projection
    size_t k_off = 0, v_off = 0;      // ATTN: byte offsets into the kv pool (set by set_pools)
    size_t state_off = 0;             // GLA: byte offset into the state pool
};

}  // namespace b200

using namespace b200;

struct b200_hybrid {
    b200_hybrid_config_t cfg;
    std::vector<b200_hybrid_layer_t> layers;
    std::vector<char> layer_set;
    std::vector<LayerPlan> plan;
    const void *embedding = nullptr, *lm_head = nullptr;
    const float *final_norm = nullptr;
    char *kv_pool = nullptr, *state_pool = nullptr;
    int num_pages = 0, num_slots = 0;
    // scratch carve-up
    char *scratch = nullptr;
    float *x = nullptr, *f32a = nullptr, *f32b = nullptr, *xn = nullptr;
    void *h = nullptr, *proj = nullptr, *mix = nullptr, *mix2 = nullptr, *y = nullptr, *xg = nullptr, *u = nullptr, *yrows = nullptr, *us = nullptr,
         *ys = nullptr;
    int *meta = nullptr, *moe_i = nullptr;
    float *moe_f = nullptr;
    std::vector<int> host_meta;
};

namespace {

struct Carve {
    size_t x, f32a, f32b, xn, h, proj, mix, y, xg, u, yrows, us, ys, meta, moe_i, moe_f, total;
};

int max_rows_of(const b200_hybrid_config_t &c, const b200_hybrid_layer_t &l) {
    const int pairs = c.max_tokens * l.top;
    return ((pairs + 127) / 128 + l.experts) * 128;  // the larger of the two row-tile sizes
}

int n_in_of(const b200_hybrid_layer_t &l) {
    if (l.mixer == B200_MIXER_ATTN_CHUNKED) return (2 * l.heads + l.kv_heads) * l.dim;
    return 2 * l.heads * l.dim + 2 * l.heads * l.vdim + l.decay_rank;
}

Carve carve(const b200_hybrid *m) {
    const b200_hybrid_config_t &c = m->cfg;
    const size_t T = (size_t)c.max_tokens, es = c.dtype == B200_F32 ? 4 : 2;
    size_t n_in = 1, n_mix = 1, n_f32 = 1, rows = 0, ff = 1, sff = 1, experts = 1, top = 1;
    for (int i = 0; i < c.num_layers; ++i) {
        if (!m->layer_set[i]) continue;
        const b200_hybrid_layer_t &l = m->layers[i];
        n_in = std::max(n_in, (size_t)n_in_of(l));
        n_mix = std::max(n_mix, (size_t)l.heads * std::max(l.dim, l.vdim));
        n_f32 = std::max(n_f32, (size_t)l.heads * std::max(l.dim, l.vdim));
        if (l.mlp == B200_MLP_MOE) {
            rows = std::max(rows, (size_t)max_rows_of(c, l));
            ff = std::max(ff, (size_t)l.expert_ff), sff = std::max(sff, (size_t)l.shared_ff);
            experts = std::max(experts, (size_t)l.experts), top = std::max(top, (size_t)l.top);
            n_f32 = std::max(n_f32, (size_t)l.experts + 1);
        }
    }
    Carve k;
    k.x = align256(T * c.width * 4);
    k.f32a = align256(T * n_f32 * 4);
    k.f32b = align256(T * n_f32 * 4);
    k.xn = align256(T * c.width * 4);
    k.h = align256(T * c.width * es);
    k.proj = align256(T * n_in * es);
    k.mix = align256(T * n_mix * es);
    k.y = align256(T * c.width * es);
    k.xg = align256(rows * c.width * es);
    k.u = align256(rows * ff * es);
    k.yrows = align256(rows * c.width * es);
    k.us = align256(T * sff * es);
    k.ys = align256(T * c.width * es);
    // meta: attention tiles [4 * (T/64 + S), padded] | ids | tok_seq | tok_pos | want | short-portion token list [T each] | seq_start [S+1] |
    //       pos0 | slot [S each] | block table [S * mpps]
    k.meta = align256((4 * (T / 64 + (size_t)c.max_seqs + 1) + 5 * T + 3 * (size_t)c.max_seqs + 1 + (size_t)c.max_seqs * c.max_pages_per_seq) * 4);
    // moe ints: sel_expert | pair_row [T*top each] | row_token [rows] | tile_expert [rows / tile] | n_tiles
    k.moe_i = align256((2 * T * top + rows + rows / kMoeTileM + 4) * 4);
    // moe floats: sel_weight [T*top] | row_weight [rows] | shared_gate [T]
    k.moe_f = align256((T * top + rows + T) * 4);
    k.total = k.x + k.f32a + k.f32b + k.xn + k.h + k.proj + 2 * k.mix + k.y + k.xg + k.u + k.yrows + k.us + k.ys + k.meta + k.moe_i + k.moe_f;
    return k;
}

int linear(const b200_hybrid *m, const void *x, const void *w, void *y, int M, int K, int N, cudaStream_t st) {
    return b200_linear(x, w, nullptr, nullptr, y, M, K, N, m->cfg.dtype, B200_W_DENSE, B200_LAYOUT_NK, 0, (b200_stream_t)st);
}

}  // namespace

extern "C" {

b200_hybrid_t *b200_hybrid_create(const b200_hybrid_config_t *cfg) {
    if (!cfg || cfg->width <= 0 || cfg->vocab <= 0 || cfg->num_layers <= 0 || cfg->max_tokens <= 0 || cfg->max_seqs <= 0 ||
        cfg->max_pages_per_seq <= 0 || (cfg->dtype != B200_F32 && cfg->dtype != B200_F16 && cfg->dtype != B200_BF16)) {
        set_error("hybrid_create: bad configuration");
        return nullptr;
    }
    b200_hybrid *m = new (std::nothrow) b200_hybrid();
    if (!m) return nullptr;
    m->cfg = *cfg;
    m->layers.resize(cfg->num_layers);
    m->layer_set.assign(cfg->num_layers, 0);
    m->plan.resize(cfg->num_layers);
    return m;
}

void b200_hybrid_destroy(b200_hybrid_t *m) { delete m; }

int b200_hybrid_set_layer(b200_hybrid_t *m, int layer, const b200_hybrid_layer_t *w) {
    B200_REQUIRE(m && w, "hybrid_set_layer: null argument");
    B200_REQUIRE(layer >= 0 && layer < m->cfg.num_layers, "hybrid_set_layer: layer %d outside [0, %d)", layer, m->cfg.num_layers);
    B200_REQUIRE(w->mixer == B200_MIXER_ATTN_CHUNKED || w->mixer == B200_MIXER_GLA, "hybrid_set_layer: unknown mixer kind %d", w->mixer);
    B200_REQUIRE(w->heads > 0 && w->dim > 0 && w->w_in && w->w_out && w->norm1, "hybrid_set_layer: mixer sizes / weights missing");
    if (w->mixer == B200_MIXER_ATTN_CHUNKED) {
        B200_REQUIRE(w->kv_heads > 0 && w->heads % w->kv_heads == 0, "hybrid_set_layer: heads %d not a multiple of kv_heads %d", w->heads, w->kv_heads);
        B200_REQUIRE(w->vdim == w->dim, "hybrid_set_layer: this attention's values are its keys: vdim %d must equal dim %d", w->vdim, w->dim);
        B200_REQUIRE(w->chunk >= 0, "hybrid_set_layer: negative chunk");
    } else {
        B200_REQUIRE(w->vdim > 0 && w->decay_rank > 0 && w->tau > 0.0f && w->w_decay && w->out_norm, "hybrid_set_layer: gla sizes / weights missing");
    }
    B200_REQUIRE(w->mlp == B200_MLP_NONE || w->mlp == B200_MLP_MOE, "hybrid_set_layer: unknown feed-forward kind %d", w->mlp);
    if (w->mlp == B200_MLP_MOE) {
        B200_REQUIRE(w->experts > 0 && w->top > 0 && w->top <= w->experts && w->expert_ff > 0 && w->shared_ff >= 0,
                     "hybrid_set_layer: bad expert counts");
        B200_REQUIRE(w->w_router && w->w_up && w->w_down && w->norm2, "hybrid_set_layer: expert weights missing");
        B200_REQUIRE(w->shared_ff == 0 || (w->w_shared_up && w->w_shared_down), "hybrid_set_layer: shared expert weights missing");
        B200_REQUIRE(w->act >= B200_ACT_RELU2 && w->act <= B200_ACT_GELU_TANH, "hybrid_set_layer: unknown activation %d", w->act);
    }
    m->layers[layer] = *w;
    m->layer_set[layer] = 1;
    m->plan[layer].n_in = n_in_of(*w);
    m->scratch = nullptr;  // sizes may have changed
    return B200_OK;
}

int b200_hybrid_set_io(b200_hybrid_t *m, const void *embedding, const float *final_norm, const void *lm_head) {
    B200_REQUIRE(m && embedding && final_norm && lm_head, "hybrid_set_io: null argument");
    m->embedding = embedding, m->final_norm = final_norm, m->lm_head = lm_head;
    return B200_OK;
}

size_t b200_hybrid_scratch_bytes(const b200_hybrid_t *m) { return m ? carve(m).total : 0; }

int b200_hybrid_set_scratch(b200_hybrid_t *m, void *ptr, size_t bytes) {
    B200_REQUIRE(m && ptr, "hybrid_set_scratch: null argument");
    B200_REQUIRE(((uintptr_t)ptr & 255) == 0, "hybrid_set_scratch: pointer must be 256-byte aligned");
    for (int i = 0; i < m->cfg.num_layers; ++i) B200_REQUIRE(m->layer_set[i], "hybrid_set_scratch: layer %d not set", i);
    const Carve k = carve(m);
    B200_REQUIRE(bytes >= k.total, "hybrid_set_scratch: need %zu bytes, got %zu", k.total, bytes);
    char *p = (char *)ptr;
    m->scratch = p;
    m->x = (float *)p, p += k.x;
    m->f32a = (float *)p, p += k.f32a;
    m->f32b = (float *)p, p += k.f32b;
    m->xn = (float *)p, p += k.xn;
    m->h = p, p += k.h;
    m->proj = p, p += k.proj;
    m->mix = p, p += k.mix;
    m->mix2 = p, p += k.mix;
    m->y = p, p += k.y;
    m->xg = p, p += k.xg;
    m->u = p, p += k.u;
    m->yrows = p, p += k.yrows;
    m->us = p, p += k.us;
    m->ys = p, p += k.ys;
    m->meta = (int *)p, p += k.meta;
    m->moe_i = (int *)p, p += k.moe_i;
    m->moe_f = (float *)p, p += k.moe_f;
    return B200_OK;
}

size_t b200_hybrid_kv_pool_bytes(const b200_hybrid_t *m, int num_pages) {
    if (!m || num_pages <= 0) return 0;
    const size_t es = m->cfg.dtype == B200_F32 ? 4 : 2;
    size_t total = 0;
    for (int i = 0; i < m->cfg.num_layers; ++i)
        if (m->layer_set[i] && m->layers[i].mixer == B200_MIXER_ATTN_CHUNKED)
            total += 2 * align256((size_t)num_pages * m->layers[i].kv_heads * kPageH * m->layers[i].dim * es);
    return total ? total : 256;
}

size_t b200_hybrid_state_pool_bytes(const b200_hybrid_t *m, int num_slots) {
    if (!m || num_slots <= 0) return 0;
    size_t total = 0;
    for (int i = 0; i < m->cfg.num_layers; ++i)
        if (m->layer_set[i] && m->layers[i].mixer == B200_MIXER_GLA)
            total += align256((size_t)num_slots * m->layers[i].heads * m->layers[i].dim * m->layers[i].vdim * 4);
    return total ? total : 256;
}

int b200_hybrid_set_pools(b200_hybrid_t *m, void *kv_pool, int num_pages, void *state_pool, int num_slots) {
    B200_REQUIRE(m && kv_pool && state_pool && num_pages > 0 && num_slots > 0, "hybrid_set_pools: bad argument");
    B200_REQUIRE(((uintptr_t)kv_pool & 255) == 0 && ((uintptr_t)state_pool & 255) == 0, "hybrid_set_pools: pools must be 256-byte aligned");
    const size_t es = m->cfg.dtype == B200_F32 ? 4 : 2;
    size_t kv = 0, stt = 0;
    for (int i = 0; i < m->cfg.num_layers; ++i) {
        B200_REQUIRE(m->layer_set[i], "hybrid_set_pools: layer %d not set", i);
        const b200_hybrid_layer_t &l = m->layers[i];
        if (l.mixer == B200_MIXER_ATTN_CHUNKED) {
            const size_t one = align256((size_t)num_pages * l.kv_heads * kPageH * l.dim * es);
            m->plan[i].k_off = kv, m->plan[i].v_off = kv + one, kv += 2 * one;
        } else {
            m->plan[i].state_off = stt, stt += align256((size_t)num_slots * l.heads * l.dim * l.vdim * 4);
        }
    }
    m->kv_pool = (char *)kv_pool, m->state_pool = (char *)state_pool, m->num_pages = num_pages, m->num_slots = num_slots;
    return B200_OK;
}

int b200_hybrid_forward(b200_hybrid_t *m, const b200_hybrid_batch_t *b, float *logits, float *layer_trace, b200_stream_t stream) {
    B200_REQUIRE(m && b, "hybrid_forward: null argument");
    if (!m->scratch || !m->kv_pool || !m->embedding) {
        set_error("hybrid_forward: scratch, pools or embedding / head not set");
        return B200_ERR_STATE;
    }
    const b200_hybrid_config_t &c = m->cfg;
    const int NT = b->n_tokens, S = b->n_seqs, W = b->n_want, mpps = c.max_pages_per_seq;
    B200_REQUIRE(NT >= 0 && NT <= c.max_tokens && S >= 0 && S <= c.max_seqs && W >= 0 && W <= NT, "hybrid_forward: %d tokens / %d sequences / %d wanted rows outside the engine's limits (%d, %d)",
                 NT, S, W, c.max_tokens, c.max_seqs);
    if (NT == 0) return B200_OK;
    B200_REQUIRE(b->token_ids && b->seq_start && b->seq_pos0 && b->seq_slot && b->block_table && (W == 0 || (b->want_rows && logits)),
                 "hybrid_forward: null batch array");
    B200_REQUIRE(b->seq_start[0] == 0 && b->seq_start[S] == NT, "hybrid_forward: seq_start must run from 0 to n_tokens");

    // ---- batch description: checked on the host, shipped in one copy
    std::vector<int> &hm = m->host_meta;
    const size_t n_tile_ints = 4 * ((size_t)NT / 64 + S + 1);
    hm.assign(n_tile_ints + (size_t)5 * NT + 3 * S + 1 + (size_t)S * mpps, 0);
    int *h_tiles = hm.data(), *h_ids = h_tiles + n_tile_ints, *h_seq = h_ids + NT, *h_pos = h_seq + NT, *h_want = h_pos + NT, *h_short = h_want + NT,
        *h_start = h_short + NT, *h_pos0 = h_start + S + 1, *h_slot = h_pos0 + S, *h_bt = h_slot + S;
    // prompt portions go to the tensor-core attention in tiles of <= 64 consecutive tokens, short ones (decoded tokens) to the per-token kernel
    constexpr int kShortPortion = 8;
    int n_tiles = 0, n_short = 0, gla_kinds = 0;
    for (int s = 0; s < S; ++s) {
        const int t0 = b->seq_start[s], t1 = b->seq_start[s + 1];
        gla_kinds |= t1 - t0 == 1 ? kGlaOneToken : (t1 - t0 > 1 ? kGlaManyTokens : 0);
        B200_REQUIRE(t1 >= t0 && b->seq_pos0[s] >= 0, "hybrid_forward: bad portion of sequence %d", s);
        B200_REQUIRE(b->seq_slot[s] >= 0 && b->seq_slot[s] < m->num_slots, "hybrid_forward: state slot %d outside [0, %d)", b->seq_slot[s], m->num_slots);
        for (int s2 = 0; s2 < s; ++s2) B200_REQUIRE(b->seq_slot[s2] != b->seq_slot[s], "hybrid_forward: state slot %d given to two sequences", b->seq_slot[s]);
        const int last = b->seq_pos0[s] + (t1 - t0) - 1;
        B200_REQUIRE(last < mpps * kPageH, "hybrid_forward: position %d exceeds a block-table row (%d pages)", last, mpps);
        for (int p = 0; p <= last / kPageH && t1 > t0; ++p) {
            const int page = b->block_table[(size_t)s * mpps + p];
            B200_REQUIRE(page >= 0 && page < m->num_pages, "hybrid_forward: sequence %d holds no page for positions %d..", s, p * kPageH);
        }
        for (int t = t0; t < t1; ++t) h_seq[t] = s, h_pos[t] = b->seq_pos0[s] + (t - t0);
        if (t1 - t0 < kShortPortion) {
            for (int t = t0; t < t1; ++t) h_short[n_short++] = t;
        } else {
            for (int t = t0; t < t1; t += 64, ++n_tiles) {
                int *tl = h_tiles + 4 * n_tiles;
                tl[0] = s, tl[1] = t, tl[2] = std::min(64, t1 - t), tl[3] = h_pos[t];
            }
        }
        h_start[s] = t0, h_pos0[s] = b->seq_pos0[s], h_slot[s] = b->seq_slot[s];
        for (int p = 0; p < mpps; ++p) h_bt[(size_t)s * mpps + p] = b->block_table[(size_t)s * mpps + p];
    }
    h_start[S] = NT;
    for (int t = 0; t < NT; ++t) {
        B200_REQUIRE(b->token_ids[t] >= 0 && b->token_ids[t] < c.vocab, "hybrid_forward: token id %d outside the vocabulary", b->token_ids[t]);
        h_ids[t] = b->token_ids[t];
    }
    for (int i = 0; i < W; ++i) {
        B200_REQUIRE(b->want_rows[i] >= 0 && b->want_rows[i] < NT, "hybrid_forward: wanted row %d outside the batch", b->want_rows[i]);
        h_want[i] = b->want_rows[i];
    }
    cudaStream_t st = as_stream(stream);
    NvtxRange range("hybrid_forward");
    if (cudaMemcpyAsync(m->meta, hm.data(), hm.size() * sizeof(int), cudaMemcpyHostToDevice, st) != cudaSuccess) return cuda_status("hybrid_forward meta copy");
    const int *d_tiles = m->meta, *d_ids = d_tiles + n_tile_ints, *d_seq = d_ids + NT, *d_pos = d_seq + NT, *d_want = d_pos + NT, *d_short = d_want + NT,
              *d_start = d_short + NT, *d_pos0 = d_start + S + 1, *d_slot = d_pos0 + S, *d_bt = d_slot + S;

    const int dt = c.dtype, width = c.width;
    const bool f32 = dt == B200_F32;
    int rc;
#define RUN(expr)                    \
    do {                             \
        rc = (expr);                 \
        if (rc != B200_OK) return rc; \
    } while (0)
    // 16-bit engines: every kernel that writes the residual stream also writes its 16-bit copy h, which the next projections read
    B200_DISPATCH_DTYPE(dt, { embed_f32_kernel<T><<<NT, 128, 0, st>>>(d_ids, (const T *)m->embedding, m->x, f32 ? nullptr : (T *)m->h, width, c.vocab); });
    auto cast_x = [&]() -> const void * { return f32 ? (const void *)m->x : (const void *)m->h; };
    auto postnorm = [&](const void *y_dense, const void *y_rows, const int *pair_row, int top, const void *y_shared, const float *gate,
                        const float *g, float *trace) -> int {
        B200_DISPATCH_DTYPE(dt, {
            postnorm_residual_kernel<T><<<NT, 256, (size_t)width * sizeof(float), st>>>(m->x, (const T *)y_dense, (const T *)y_rows, pair_row, top,
                                                                                      (const T *)y_shared, gate, g, c.norm_eps, width, trace,
                                                                                      f32 ? nullptr : (T *)m->h);
        });
        return cuda_status("postnorm_residual launch");
    };

    for (int li = 0; li < c.num_layers; ++li) {
        const b200_hybrid_layer_t &l = m->layers[li];
        const LayerPlan &lp = m->plan[li];
        float *trace = (layer_trace && l.mlp == B200_MLP_NONE) ? layer_trace + (size_t)li * NT * width : nullptr;
        const void *h = cast_x();
        RUN(linear(m, h, l.w_in, m->proj, NT, width, lp.n_in, st));
        if (l.mixer == B200_MIXER_ATTN_CHUNKED) {
            const int hd = l.heads * l.dim;
            const size_t es = f32 ? 4 : 2;
            const char *gate = (const char *)m->proj + (size_t)(l.heads + l.kv_heads) * l.dim * es;
            RUN(launch_attn_qk_norm_cache(dt, m->proj, lp.n_in, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.q_norm, l.k_norm, c.norm_eps,
                                          d_seq, d_pos, d_bt, mpps, NT, l.heads, l.kv_heads, l.dim, st));
            const int max_keys = l.chunk > 0 ? l.chunk : mpps * kPageH;
            if (chunked_attention_tiles_supported(dt, l.dim, lp.n_in)) {
                RUN(launch_chunked_attention_tiles(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_tiles,
                                                   n_tiles, d_bt, mpps, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, st));
                RUN(launch_chunked_attention(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_seq, d_pos,
                                             d_bt, mpps, n_short, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, max_keys, st, d_short));
            } else {
                RUN(launch_chunked_attention(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_seq, d_pos,
                                             d_bt, mpps, NT, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, max_keys, st));
            }
            RUN(linear(m, m->mix2, l.w_out, m->y, NT, hd, width, st));
        } else {
            const int hd = l.heads * l.dim, hv = l.heads * l.vdim;
            const size_t es = f32 ? 4 : 2;
            const char *gate = (const char *)m->proj + (size_t)(2 * hd + hv) * es;
            RUN(launch_gla_decay(dt, m->proj, lp.n_in, 2 * hd + 2 * hv, l.w_decay, l.decay_bias, l.tau, m->f32a, NT, l.decay_rank, hd, st));
            RUN(launch_gla_recurrent(dt, m->proj, lp.n_in, m->f32a, (float *)(m->state_pool + lp.state_off), m->f32b, d_start, d_pos0, d_slot, S,
                                     l.heads, l.dim, l.vdim, st, gla_kinds));
            RUN(launch_gla_output(dt, m->f32b, l.out_norm, c.norm_eps, gate, lp.n_in, m->mix2, NT, l.heads, l.vdim, st));
            RUN(linear(m, m->mix2, l.w_out, m->y, NT, hv, width, st));
        }
        RUN(postnorm(m->y, nullptr, nullptr, 0, nullptr, nullptr, l.norm1, trace));
        if (l.mlp == B200_MLP_MOE) {
            trace = layer_trace ? layer_trace + (size_t)li * NT * width : nullptr;
            const int pairs = NT * l.top;
            // prompt-sized batches of a 16-bit engine: 128-row tiles on the tcgen05 grouped GEMM; otherwise 64-row tiles on mma.sync / SIMT
            const bool tc = !f32 && pairs >= 1024 && width % 8 == 0 && l.expert_ff % 8 == 0 && width >= 64 && l.expert_ff >= 64;
            const int tile = tc ? 128 : kMoeTileM;
            const int max_rows = ((pairs + tile - 1) / tile + std::min(l.experts, pairs)) * tile;
            const int max_tiles = max_rows / tile;
            int *sel_expert = m->moe_i, *pair_row = sel_expert + pairs, *row_token = pair_row + pairs, *tile_expert = row_token + max_rows,
                *n_tiles = tile_expert + max_tiles;
            float *sel_weight = m->moe_f, *row_weight = sel_weight + pairs, *shared_gate = row_weight + max_rows;
            const void *h2 = cast_x();
            // router logits + shared gate, fp32: 16-bit engines multiply the 16-bit copy of x on the tensor cores (products of 16-bit values
            // are exact in fp32 and the sums are fp32), others -- and widths the tensor-core kernel does not take -- the fp32 kernel
            // (a decode batch is a single 64-row tile there -- one CTA walking all of K -- so few tokens take the fp32 kernel as well)
            rc = NT >= 64 ? launch_dense_f32out(dt, h2, l.w_router, m->f32a, NT, l.experts + 1, width, st) : B200_ERR_UNSUPPORTED;
            if (rc == B200_ERR_UNSUPPORTED) rc = launch_proj_f32(B200_F32, m->x, width, dt, l.w_router, nullptr, m->f32a, l.experts + 1, NT, l.experts + 1, width, st);
            if (rc != B200_OK) return rc;
            RUN(launch_moe_route_sigmoid(m->f32a, l.experts + 1, sel_expert, sel_weight, shared_gate, NT, l.experts, l.top, st));
            RUN(launch_moe_plan(sel_expert, sel_weight, row_token, row_weight, tile_expert, pair_row, n_tiles, NT, l.experts, l.top, tile, st));
            RUN(launch_moe_gather(dt, m->x, row_token, row_weight, m->xg, n_tiles, max_rows, width, tile, st));
            if (tc) {
                RUN(launch_gemm_tc_grouped(m->xg, l.w_up, m->u, max_rows, l.expert_ff, width, l.experts, tile_expert, n_tiles, l.act, dt, st));
                RUN(launch_gemm_tc_grouped(m->u, l.w_down, m->yrows, max_rows, width, l.expert_ff, l.experts, tile_expert, n_tiles, -1, dt, st));
            } else {
                RUN(launch_moe_grouped_gemm(dt, m->xg, l.w_up, m->u, tile_expert, n_tiles, max_tiles, l.expert_ff, width, l.act, st));
                RUN(launch_moe_grouped_gemm(dt, m->u, l.w_down, m->yrows, tile_expert, n_tiles, max_tiles, width, l.expert_ff, -1, st));
            }
            if (l.shared_ff > 0) {
                RUN(linear(m, h2, l.w_shared_up, m->us, NT, width, l.shared_ff, st));
                RUN(launch_activation(dt, m->us, (size_t)NT * l.shared_ff, l.act, st));
                RUN(linear(m, m->us, l.w_shared_down, m->ys, NT, l.shared_ff, width, st));
            }
            RUN(postnorm(nullptr, m->yrows, pair_row, l.top, l.shared_ff > 0 ? m->ys : nullptr, shared_gate, l.norm2, trace));
        }
    }
    if (W > 0) {
        // the wanted rows only: final norm (fp32 and, for 16-bit engines, a 16-bit copy in h), then the LM head with fp32 logits
        B200_DISPATCH_DTYPE(dt, { final_norm_rows_kernel<T><<<W, 256, 0, st>>>(m->x, d_want, m->final_norm, c.norm_eps, m->xn, f32 ? nullptr : (T *)m->h, width); });
        rc = launch_dense_f32out(dt, m->h, m->lm_head, logits, W, c.vocab, width, st);
        if (rc == B200_ERR_UNSUPPORTED) rc = launch_proj_f32(B200_F32, m->xn, width, dt, m->lm_head, nullptr, logits, c.vocab, W, c.vocab, width, st);
        if (rc != B200_OK) return rc;
    }
#undef RUN
    return cuda_status("hybrid_forward");
}
}
