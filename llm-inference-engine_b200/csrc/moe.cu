// moe.cu -- mixture-of-experts feed-forward for ragged token batches.  (Row tiles are 64 rows for the kernels of this file, 128 for the
// tcgen05 grouped GEMM of gemm_tc.cu, which serves prompt-sized batches of 16-bit engines; the engine chooses per call.)
//   route:   scores = sigmoid(router logits) (fp32); the `top` largest are chosen, their scores ARE the weights (no renormalisation);
//            a separate sigmoid gate scales the shared expert.
//   plan:    the (token, choice) pairs are grouped by expert; every expert's rows are padded to whole tiles of kMoeTileM rows so that a
//            tile of the grouped GEMM belongs to exactly one expert.  Done on the device: the host never learns the counts, it launches
//            the worst-case number of tiles and the surplus CTAs leave at once.
//   gather:  row <- T(weight * x[token])  -- the weight multiplies the expert's input, which matters for a non-linear expert;
//   grouped GEMM (x2): up with the activation in the epilogue, then down.
// A second router form (softmax): scores = softmax(router logits) over all router outputs; the choice is made on score + a per-expert bias,
// the weights are the chosen experts' scores divided by their sum and multiply the expert's OUTPUT; router outputs past the real experts
// are identity experts (they return their input and own no rows of the grouped GEMM); experts may be gated: act(gate rows) * up rows.
// The sum over a token's experts, the shared expert and the post-norm are one kernel of the engine (hybrid.cu).
#include "hybrid_ops.cuh"

#include <algorithm>

namespace b200 {

// one warp per token
__global__ void moe_route_sigmoid_kernel(const float *__restrict__ logits, int ld, int *__restrict__ sel_expert, float *__restrict__ sel_weight,
                                         float *__restrict__ shared_gate, int tokens, int experts, int top) {
    const int t = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const float *z = logits + (size_t)t * ld;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            bool taken = false;
            for (int p = 0; p < k; ++p) taken |= sel_expert[(size_t)t * top + p] == e;
            const float v = z[e];
            if (!taken && (v > best || (v == best && e < bi))) best = v, bi = e;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi;
        }
        if (lane == 0) {
            sel_expert[(size_t)t * top + k] = bi;
            sel_weight[(size_t)t * top + k] = 1.0f / (1.0f + expf(-best));  // sigmoid is monotone: the largest logit has the largest score
        }
        __syncwarp();
    }
    if (lane == 0 && shared_gate) shared_gate[t] = 1.0f / (1.0f + expf(-z[experts]));
}

// one warp per token; `outputs` router outputs (real experts first, then identity experts)
__global__ void moe_route_softmax_kernel(const float *__restrict__ logits, int ld, const float *__restrict__ bias, int *__restrict__ sel_expert,
                                         float *__restrict__ sel_weight, int tokens, int outputs, int top) {
    const int t = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const float *z = logits + (size_t)t * ld;
    float mx = -INFINITY;
    for (int e = lane; e < outputs; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float den = 0.0f;
    for (int e = lane; e < outputs; e += 32) den += expf(z[e] - mx);
    den = warp_sum(den);
    const float inv = 1.0f / den;
    float chosen_sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY, best_s = 0.0f;
        int bi = 0x7fffffff;
        for (int e = lane; e < outputs; e += 32) {
            bool taken = false;
            for (int p = 0; p < k; ++p) taken |= sel_expert[(size_t)t * top + p] == e;
            const float sc = expf(z[e] - mx) * inv;
            const float v = sc + (bias ? bias[e] : 0.0f);
            if (!taken && (v > best || (v == best && e < bi))) best = v, bi = e, best_s = sc;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, best_s, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) best = ov, bi = oi, best_s = os;
        }
        chosen_sum += best_s;
        if (lane == 0) {
            sel_expert[(size_t)t * top + k] = bi;
            sel_weight[(size_t)t * top + k] = best_s;
        }
        __syncwarp();
    }
    const float norm = 1.0f / (chosen_sum + 1e-20f);
    for (int k = lane; k < top; k += 32) sel_weight[(size_t)t * top + k] *= norm;
}

// one CTA.  Shared: count[E] | offset[E+1] | cursor[E]
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int *__restrict__ sel_expert, const float *__restrict__ sel_weight, int *__restrict__ row_token, float *__restrict__ row_weight,
                int *__restrict__ tile_expert, int *__restrict__ pair_row, int *__restrict__ n_tiles, int pairs, int experts, int top, int tile) {
    // choices >= experts (identity experts) own no row: pair_row = -1
    extern __shared__ int si[];
    int *count = si, *offset = si + experts, *cursor = offset + experts + 1;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0, cursor[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x)
        if (sel_expert[p] < experts) atomicAdd(&count[sel_expert[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            offset[e] = at;
            const int tiles = (count[e] + tile - 1) / tile;
            for (int i = 0; i < tiles; ++i) tile_expert[at / tile + i] = e;
            at += tiles * tile;
        }
        offset[experts] = at;
        *n_tiles = at / tile;
    }
    __syncthreads();
    const int rows = offset[experts];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) row_token[r] = -1, row_weight[r] = 0.0f;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = sel_expert[p];
        if (e >= experts) {
            pair_row[p] = -1;
            continue;
        }
        const int r = offset[e] + atomicAdd(&cursor[e], 1);
        row_token[r] = p / top;
        row_weight[r] = sel_weight[p];
        pair_row[p] = r;
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const float *__restrict__ x, const int *__restrict__ row_token, const float *__restrict__ row_weight, T *__restrict__ xg,
                  const int *__restrict__ n_tiles, int width, int tile) {
    const int r = blockIdx.x;
    if (r >= *n_tiles * tile) return;
    const int t = row_token[r];
    const float w = row_weight[r];
    constexpr int V = Elem<T>::kVec;
    if (width % V == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(xg)) & 15) == 0) {  // 16-byte pieces of the output row
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
            float f[V];
#pragma unroll
            for (int e = 0; e < V; e += 4) {
                const float4 a = t >= 0 ? *reinterpret_cast<const float4 *>(x + (size_t)t * width + c + e) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                f[e] = w * a.x, f[e + 1] = w * a.y, f[e + 2] = w * a.z, f[e + 3] = w * a.w;
            }
            if (t < 0) {
#pragma unroll
                for (int e = 0; e < V; ++e) f[e] = 0.0f;  // padding rows are exact zeros whatever their weight slot holds
            }
            st_v4(xg + (size_t)r * width + c, pack16<T>(f));
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        xg[(size_t)r * width + c] = Elem<T>::from_f(t >= 0 ? w * x[(size_t)t * width + c] : 0.0f);
}

// xg[row, :] = h[token[row], :] (zeros for padding rows): the expert reads the token's row as it is, the weight goes on its output
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const T *__restrict__ h, const int *__restrict__ row_token, T *__restrict__ xg, const int *__restrict__ n_tiles, int width,
                       int tile) {
    const int r = blockIdx.x;
    if (r >= *n_tiles * tile) return;
    const int t = row_token[r];
    constexpr int V = Elem<T>::kVec;
    if (width % V == 0 && ((reinterpret_cast<size_t>(h) | reinterpret_cast<size_t>(xg)) & 15) == 0) {
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V)
            st_v4(xg + (size_t)r * width + c, t >= 0 ? ld_v4(h + (size_t)t * width + c) : make_uint4(0, 0, 0, 0));
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) xg[(size_t)r * width + c] = t >= 0 ? h[(size_t)t * width + c] : Elem<T>::from_f(0.0f);
}

// out[r, c] = act(in[r, c]) * in[r, inner + c] for rows r < *n_tiles * tile (all `rows` when n_tiles is NULL); in [rows, 2 * inner].
// One 16-byte piece of the output per thread when the rows start on 16-byte boundaries, else one element.
template <typename T>
__global__ void gated_activation_kernel(const T *__restrict__ in, T *__restrict__ out, int rows, int inner, int act, const int *__restrict__ n_tiles,
                                        int tile) {
    constexpr int V = Elem<T>::kVec;
    const int live = n_tiles ? min(rows, *n_tiles * tile) : rows;
    if (inner % V == 0 && ((reinterpret_cast<size_t>(in) | reinterpret_cast<size_t>(out)) & 15) == 0) {
        const int per_row = inner / V;
        const size_t n = (size_t)live * per_row;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
            const size_t r = i / per_row, c = (i - r * per_row) * V;
            float g[V], u[V];
            unpack16<T>(ld_v4(in + r * 2 * inner + c), g);
            unpack16<T>(ld_v4(in + r * 2 * inner + inner + c), u);
#pragma unroll
            for (int e = 0; e < V; ++e) g[e] = act_apply(g[e], act) * u[e];
            st_v4(out + r * inner + c, pack16<T>(g));
        }
        return;
    }
    const size_t n = (size_t)live * inner;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inner, c = i - r * inner;
        const float g = Elem<T>::to_f(in[r * 2 * inner + c]), u = Elem<T>::to_f(in[r * 2 * inner + inner + c]);
        out[i] = Elem<T>::from_f(act_apply(g, act) * u);
    }
}

// in place: x[r, c] = act(x[r, c] + bias[c]) (bias may be NULL, act < 0: none); 16-byte pieces when the rows start on 16-byte boundaries
template <typename T>
__global__ void bias_activation_kernel(T *__restrict__ x, const float *__restrict__ bias, size_t rows, int cols, int act) {
    constexpr int V = Elem<T>::kVec;
    if (cols % V == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(bias)) & 15) == 0) {
        const int per_row = cols / V;
        const size_t n = rows * per_row;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
            const int c = (int)(i % per_row) * V;
            float f[V], b[V];
            unpack16<T>(ld_v4(x + i * V), f);
#pragma unroll
            for (int e = 0; e < V; e += 4) {  // the bias in 16-byte loads: eight scalar loads per thread are eight cache wavefronts per warp
                const float4 bv = bias ? *reinterpret_cast<const float4 *>(bias + c + e) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                b[e] = bv.x, b[e + 1] = bv.y, b[e + 2] = bv.z, b[e + 3] = bv.w;
            }
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float v = f[e] + b[e];
                f[e] = act >= 0 ? act_apply(v, act) : v;
            }
            st_v4(x + i * V, pack16<T>(f));
        }
        return;
    }
    const size_t n = rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = Elem<T>::to_f(x[i]);
        if (bias) v += bias[i % cols];
        x[i] = Elem<T>::from_f(act >= 0 ? act_apply(v, act) : v);
    }
}

// SIMT grouped GEMM, 64 x 64 tile, fp32 accumulation.  The tensor-core path of the dense linears does not apply: an expert's rows are
// few (a decode batch brings one or two per expert) and the weight of a tile is chosen per tile.
constexpr int kGT = 64, kGK = 16;
template <typename T>
__global__ void __launch_bounds__(256)
moe_grouped_gemm_kernel(const T *__restrict__ a, const T *__restrict__ w, T *__restrict__ c, const int *__restrict__ tile_expert,
                        const int *__restrict__ n_tiles, int N, int K, int act) {
    if ((int)blockIdx.y >= *n_tiles) return;
    __shared__ float As[kGK][kGT + 4];
    __shared__ float Bs[kGK][kGT + 4];
    const int m0 = blockIdx.y * kMoeTileM, n0 = blockIdx.x * kGT;
    const T *wb = w + (size_t)tile_expert[blockIdx.y] * N * K;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kGK) {
        for (int i = threadIdx.x; i < kGT * kGK; i += 256) {
            const int kk = i % kGK, mm = i / kGK;
            const int k = k0 + kk;
            As[kk][mm] = k < K ? Elem<T>::to_f(a[(size_t)(m0 + mm) * K + k]) : 0.0f;
            const int n = n0 + mm;
            Bs[kk][mm] = (n < N && k < K) ? Elem<T>::to_f(wb[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (n < N) c[(size_t)m * N + n] = Elem<T>::from_f(act >= 0 ? act_apply(acc[i][j], act) : acc[i][j]);
        }
}

// Tensor-core grouped GEMM for 16-bit engines (K a multiple of 8): CTA tile 64 rows (one expert's tile) x 128 columns, K in steps of 64
// through a three-stage cp.async ring, four warps of 32 x 64 on mma.sync.m16n8k16, fp32 accumulators, activation in the epilogue.
constexpr int kMN = 128, kMK = 64, kMStages = 3;
__device__ __forceinline__ void moe_cp16(void *smem, const void *gmem, bool live) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = live ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ int moe_swz(int row, int col) { return row * kMK + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)); }
template <typename T> __device__ __forceinline__ void moe_mma(float *c, const unsigned *a, unsigned b0, unsigned b1);
template <> __device__ __forceinline__ void moe_mma<__nv_bfloat16>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void moe_mma<__half>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void moe_ldsm(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}

// The same kernel serves the dense fp32-output projections of a 16-bit engine (router logits, LM head): tile_expert == NULL (one weight),
// n_tiles == NULL (every tile of the grid is live), rows >= M are zero-filled on load and not stored, TC = float.
template <typename T, typename TC>
__global__ void __launch_bounds__(128)
moe_grouped_gemm_mma_kernel(const T *__restrict__ a, const T *__restrict__ w, TC *__restrict__ c, const int *__restrict__ tile_expert,
                            const int *__restrict__ n_tiles, int M, int N, int K, int act) {
    if (n_tiles && (int)blockIdx.y >= *n_tiles) return;
    extern __shared__ __align__(16) unsigned char smraw[];
    T *As = reinterpret_cast<T *>(smraw);               // [stages][64][64]
    T *Bs = As + kMStages * kMoeTileM * kMK;            // [stages][128][64]
    const int m0 = blockIdx.y * kMoeTileM, n0 = blockIdx.x * kMN;
    const T *wb = w + (tile_expert ? (size_t)tile_expert[blockIdx.y] * N * K : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;
    const int nk = (K + kMK - 1) / kMK;
    auto load = [&](int kt, int stage) {
        const int k0 = kt * kMK;
        T *as = As + stage * kMoeTileM * kMK, *bs = Bs + stage * kMN * kMK;
        for (int i = threadIdx.x; i < kMoeTileM * 8; i += 128) {
            const int r = i >> 3, cc = (i & 7) * 8;
            const bool live = k0 + cc < K && m0 + r < M;
            moe_cp16(as + moe_swz(r, cc), a + (live ? (size_t)(m0 + r) * K + k0 + cc : 0), live);
        }
        for (int i = threadIdx.x; i < kMN * 8; i += 128) {
            const int r = i >> 3, cc = (i & 7) * 8;
            const bool live = k0 + cc < K && n0 + r < N;
            moe_cp16(bs + moe_swz(r, cc), wb + (live ? (size_t)(n0 + r) * K + k0 + cc : 0), live);
        }
    };
    for (int s = 0; s < kMStages - 1; ++s) {
        if (s < nk) load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;
    for (int kt = 0; kt < nk; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kMStages - 2) : "memory");
        __syncthreads();
        if (kt + kMStages - 1 < nk) load(kt + kMStages - 1, (kt + kMStages - 1) % kMStages);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const T *as = As + (kt % kMStages) * kMoeTileM * kMK, *bs = Bs + (kt % kMStages) * kMN * kMK;
#pragma unroll
        for (int kk = 0; kk < kMK / 16; ++kk) {
            unsigned af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                moe_ldsm(af[i][0], af[i][1], af[i][2], af[i][3], as + moe_swz(wm * 32 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                unsigned b0, b1, b2, b3;
                moe_ldsm(b0, b1, b2, b3, bs + moe_swz(wn * 64 + jp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    moe_mma<T>(acc[i][2 * jp], af[i], b0, b1);
                    moe_mma<T>(acc[i][2 * jp + 1], af[i], b2, b3);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int m = m0 + wm * 32 + i * 16 + gid + (e >> 1) * 8, n = n0 + wn * 64 + j * 8 + tig * 2 + (e & 1);
                if (n < N && m < M) c[(size_t)m * N + n] = Elem<TC>::from_f(act >= 0 ? act_apply(acc[i][j][e], act) : acc[i][j][e]);
            }
}

// y fp32 [M, N] = x [M, K] (16-bit) * w[N, K]^T on the tensor cores, fp32 accumulation and fp32 result
int launch_dense_f32out(int dtype, const void *x, const void *w, float *y, int M, int N, int K, cudaStream_t st) {
    if (M == 0) return B200_OK;
    if (dtype == B200_F32 || K % 8 != 0) return B200_ERR_UNSUPPORTED;
    const dim3 grid((N + kMN - 1) / kMN, (M + kMoeTileM - 1) / kMoeTileM);
    const size_t smem = (size_t)kMStages * (kMoeTileM + kMN) * kMK * 2;
    if (dtype == B200_BF16) {
        cudaFuncSetAttribute(moe_grouped_gemm_mma_kernel<__nv_bfloat16, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        moe_grouped_gemm_mma_kernel<__nv_bfloat16, float><<<grid, 128, smem, st>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)w, y, nullptr, nullptr, M, N, K, -1);
    } else {
        cudaFuncSetAttribute(moe_grouped_gemm_mma_kernel<__half, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        moe_grouped_gemm_mma_kernel<__half, float><<<grid, 128, smem, st>>>((const __half *)x, (const __half *)w, y, nullptr, nullptr, M, N, K, -1);
    }
    return cuda_status("dense_f32out launch");
}

// one 16-byte piece per thread; the last n % kVec elements (and everything, if x is not 16-byte aligned) one by one
template <typename T>
__global__ void activation_kernel(T *__restrict__ x, size_t n, int act, size_t n_vec) {
    constexpr int V = Elem<T>::kVec;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_vec) {
        float f[V];
        unpack16<T>(ld_v4(x + i * V), f);
#pragma unroll
        for (int e = 0; e < V; ++e) f[e] = act_apply(f[e], act);
        st_v4(x + i * V, pack16<T>(f));
    } else {
        const size_t j = n_vec * V + (i - n_vec);
        if (j < n) x[j] = Elem<T>::from_f(act_apply(Elem<T>::to_f(x[j]), act));
    }
}

int launch_moe_route_sigmoid(const float *logits, int ld, int *sel_expert, float *sel_weight, float *shared_gate, int tokens,
                             int experts, int top, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    moe_route_sigmoid_kernel<<<(tokens + 3) / 4, 128, 0, st>>>(logits, ld, sel_expert, sel_weight, shared_gate, tokens, experts, top);
    return cuda_status("moe_route launch");
}

int launch_moe_route_softmax(const float *logits, int ld, const float *bias, int *sel_expert, float *sel_weight, int tokens, int outputs,
                             int top, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    moe_route_softmax_kernel<<<(tokens + 3) / 4, 128, 0, st>>>(logits, ld, bias, sel_expert, sel_weight, tokens, outputs, top);
    return cuda_status("moe_route (softmax) launch");
}

int launch_moe_gather_rows(int dtype, const void *h, const int *row_token, void *xg, const int *n_tiles, int max_rows, int width, int tile,
                           cudaStream_t st) {
    if (max_rows == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, { moe_gather_rows_kernel<T><<<max_rows, 128, 0, st>>>((const T *)h, row_token, (T *)xg, n_tiles, width, tile); });
    return cuda_status("moe_gather_rows launch");
}

int launch_gated_activation(int dtype, const void *in, void *out, int rows, int inner, int act, const int *n_tiles, int tile, cudaStream_t st) {
    if (rows == 0 || inner == 0) return B200_OK;
    const size_t n = (size_t)rows * inner / 4;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>((n + 255) / 256, 148 * 16));
    B200_DISPATCH_DTYPE(dtype, { gated_activation_kernel<T><<<grid, 256, 0, st>>>((const T *)in, (T *)out, rows, inner, act, n_tiles, tile); });
    return cuda_status("gated_activation launch");
}

int launch_bias_activation(int dtype, void *x, const float *bias, size_t rows, int cols, int act, cudaStream_t st) {
    if (rows == 0 || cols == 0) return B200_OK;
    const size_t n = rows * cols / 4;
    const unsigned grid = (unsigned)std::max<size_t>(1, std::min<size_t>((n + 255) / 256, 148 * 16));
    B200_DISPATCH_DTYPE(dtype, { bias_activation_kernel<T><<<grid, 256, 0, st>>>((T *)x, bias, rows, cols, act); });
    return cuda_status("bias_activation launch");
}

int launch_moe_plan(const int *sel_expert, const float *sel_weight, int *row_token, float *row_weight, int *tile_expert, int *pair_row,
                    int *n_tiles, int tokens, int experts, int top, int tile, cudaStream_t st) {
    moe_plan_kernel<<<1, 1024, (size_t)(3 * experts + 1) * sizeof(int), st>>>(sel_expert, sel_weight, row_token, row_weight, tile_expert,
                                                                             pair_row, n_tiles, tokens * top, experts, top, tile);
    return cuda_status("moe_plan launch");
}

int launch_moe_gather(int dtype, const float *x, const int *row_token, const float *row_weight, void *xg, const int *n_tiles,
                      int max_rows, int width, int tile, cudaStream_t st) {
    if (max_rows == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, { moe_gather_kernel<T><<<max_rows, 128, 0, st>>>(x, row_token, row_weight, (T *)xg, n_tiles, width, tile); });
    return cuda_status("moe_gather launch");
}

int launch_moe_grouped_gemm(int dtype, const void *a, const void *w, void *c, const int *tile_expert, const int *n_tiles, int max_tiles,
                            int N, int K, int act, cudaStream_t st) {
    if (max_tiles == 0) return B200_OK;
    if (dtype != B200_F32 && K % 8 == 0) {
        const dim3 grid((N + kMN - 1) / kMN, max_tiles);
        const size_t smem = (size_t)kMStages * (kMoeTileM + kMN) * kMK * 2;
        if (dtype == B200_BF16) {
            cudaFuncSetAttribute(moe_grouped_gemm_mma_kernel<__nv_bfloat16, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            moe_grouped_gemm_mma_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 128, smem, st>>>((const __nv_bfloat16 *)a, (const __nv_bfloat16 *)w, (__nv_bfloat16 *)c,
                                                                                               tile_expert, n_tiles, max_tiles * kMoeTileM, N, K, act);
        } else {
            cudaFuncSetAttribute(moe_grouped_gemm_mma_kernel<__half, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            moe_grouped_gemm_mma_kernel<__half, __half><<<grid, 128, smem, st>>>((const __half *)a, (const __half *)w, (__half *)c, tile_expert, n_tiles,
                                                                                 max_tiles * kMoeTileM, N, K, act);
        }
        return cuda_status("moe_grouped_gemm (tensor core) launch");
    }
    const dim3 grid((N + kGT - 1) / kGT, max_tiles);
    B200_DISPATCH_DTYPE(dtype, {
        moe_grouped_gemm_kernel<T><<<grid, 256, 0, st>>>((const T *)a, (const T *)w, (T *)c, tile_expert, n_tiles, N, K, act);
    });
    return cuda_status("moe_grouped_gemm launch");
}

int launch_activation(int dtype, void *x, size_t n, int act, cudaStream_t st) {
    if (n == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        const size_t n_vec = (reinterpret_cast<size_t>(x) & 15) == 0 ? n / Elem<T>::kVec : 0;
        const size_t threads = n_vec + (n - n_vec * Elem<T>::kVec);
        activation_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((T *)x, n, act, n_vec);
    });
    return cuda_status("activation launch");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route_sigmoid(const float *logits, int ld, int *sel_expert, float *sel_weight, float *shared_gate, int tokens,
                                      int experts, int top, b200_stream_t stream) {
    B200_REQUIRE(logits && sel_expert && sel_weight, "moe_route: null pointer");
    B200_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts && ld >= experts + (shared_gate ? 1 : 0), "moe_route: bad shape");
    return launch_moe_route_sigmoid(logits, ld, sel_expert, sel_weight, shared_gate, tokens, experts, top, as_stream(stream));
}

extern "C" int b200_moe_route_softmax(const float *logits, int ld, const float *bias, int *sel_expert, float *sel_weight, int tokens, int outputs,
                                      int top, b200_stream_t stream) {
    B200_REQUIRE(logits && sel_expert && sel_weight, "moe_route_softmax: null pointer");
    B200_REQUIRE(tokens >= 0 && outputs > 0 && top > 0 && top <= outputs && ld >= outputs, "moe_route_softmax: bad shape");
    return launch_moe_route_softmax(logits, ld, bias, sel_expert, sel_weight, tokens, outputs, top, as_stream(stream));
}
