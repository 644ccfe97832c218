// gla.cu -- gated linear attention (a linear-attention recurrence with a learned decay per key channel):
//     a_t = sigmoid(z_t)^(1/tau),  z_t = W2 (W1 h_t) + b           (heads x dim channels, fp32 from the low-rank projection on)
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T                           (per head, S is dim x vdim, fp32)
//     o_t = S_t^T (q_t / sqrt(dim))
//     y_t = rmsnorm_vdim(o_t) * w * silu(gate_t)                    (per head; w shared by the heads)
// The state of a sequence lives in a slot of a pool ([slots, heads, dim, vdim] fp32) between calls; a portion that starts at position 0
// starts from zero.  Columns of S are independent of one another, so a head is cut into column tiles, one CTA each: the grid is
// (vdim tiles, heads, sequences), the token loop is serial inside a CTA, the tile of S stays in shared memory for the whole portion.
// One-token portions (decoding) have a kernel of their own, laid out for one pass over the state (gla_step_kernel).
#include "hybrid_ops.cuh"

namespace b200 {

constexpr int kGlaCols = 32;     // columns of S per CTA
constexpr int kGlaThreads = 256; // 8 row groups x 32 columns

// One CTA per block of kDecayTokens tokens: a thread reads a row of the second decay matrix once and uses it for every token of the block.
constexpr int kDecayTokens = 16;
template <typename T>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const T *__restrict__ proj, int ld, int col0, const T *__restrict__ w, const float *__restrict__ bias, float inv_tau,
                 float *__restrict__ decay, int tokens, int rank, int channels) {
    extern __shared__ __align__(16) float lo[];  // [kDecayTokens][rank]: the tokens' low-rank vectors
    const int t0 = blockIdx.x * kDecayTokens;
    const int nt = min(kDecayTokens, tokens - t0);
    for (int i = threadIdx.x; i < kDecayTokens * rank; i += blockDim.x) {
        const int tt = i / rank, r = i - tt * rank;
        lo[i] = tt < nt ? Elem<T>::to_f(proj[(size_t)(t0 + tt) * ld + col0 + r]) : 0.0f;
    }
    const bool vec_w = rank % Elem<T>::kVec == 0 && (reinterpret_cast<size_t>(w) & 15) == 0;
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float z[kDecayTokens];
        const float b0 = bias ? bias[c] : 0.0f;
#pragma unroll
        for (int tt = 0; tt < kDecayTokens; ++tt) z[tt] = b0;
        const T *wr = w + (size_t)c * rank;
        if (vec_w) {
            // a row of the matrix in 16-byte pieces; four ranks per shared-memory read (one 16-byte broadcast per token)
            constexpr int V = Elem<T>::kVec;
            for (int r = 0; r < rank; r += V) {
                float wv[V];
                unpack16<T>(ld_v4(wr + r), wv);
#pragma unroll
                for (int q4 = 0; q4 < V; q4 += 4) {
#pragma unroll
                    for (int tt = 0; tt < kDecayTokens; ++tt) {
                        const float4 l = *reinterpret_cast<const float4 *>(lo + tt * rank + r + q4);
                        z[tt] = fmaf(wv[q4 + 3], l.w, fmaf(wv[q4 + 2], l.z, fmaf(wv[q4 + 1], l.y, fmaf(wv[q4], l.x, z[tt]))));
                    }
                }
            }
        } else {
            for (int r = 0; r < rank; ++r) {
                const float wv = Elem<T>::to_f(wr[r]);
#pragma unroll
                for (int tt = 0; tt < kDecayTokens; ++tt) z[tt] = fmaf(wv, lo[tt * rank + r], z[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < kDecayTokens; ++tt) {
            if (tt < nt) {
                // log sigmoid(z) = min(z, 0) - log1p(exp(-|z|));  a = exp(log sigmoid(z) / tau)
                const float ls = fminf(z[tt], 0.0f) - log1pf(expf(-fabsf(z[tt])));
                decay[(size_t)(t0 + tt) * channels + c] = expf(ls * inv_tau);
            }
        }
    }
}

// Shared memory: S[dim][kGlaCols] | q[dim] | k[dim] | a[dim] | v[kGlaCols] | part[8][kGlaCols]
template <typename T>
__global__ void __launch_bounds__(kGlaThreads)
gla_recurrent_kernel(const T *__restrict__ proj, int ld, const float *__restrict__ decay, float *__restrict__ state, float *__restrict__ o,
                     const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads,
                     int dim, int vdim, int min_tokens) {
    extern __shared__ float sm[];
    float *S = sm;
    float *qs = S + (size_t)dim * kGlaCols;
    float *ks = qs + dim;
    float *as = ks + dim;
    float *vs = as + dim;
    float *part = vs + kGlaCols;
    const int j0 = blockIdx.x * kGlaCols, h = blockIdx.y, s = blockIdx.z;
    const int col = threadIdx.x % kGlaCols, rg = threadIdx.x / kGlaCols;
    constexpr int kRowGroups = kGlaThreads / kGlaCols;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (t1 - t0 < min_tokens) return;
    const bool live = j0 + col < vdim;
    float *slot = state + (((size_t)seq_slot[s] * heads + h) * dim) * vdim;
    const bool fresh = seq_pos0[s] == 0;
    for (int i = rg; i < dim; i += kRowGroups) S[i * kGlaCols + col] = (!fresh && live) ? slot[(size_t)i * vdim + j0 + col] : 0.0f;
    const float qscale = rsqrtf((float)dim);
    const int off_k = heads * dim, off_v = 2 * heads * dim;
    for (int t = t0; t < t1; ++t) {
        const T *row = proj + (size_t)t * ld;
        __syncthreads();  // the previous token's reads of q/k/a/v/part are done
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            qs[i] = Elem<T>::to_f(row[h * dim + i]) * qscale;
            ks[i] = Elem<T>::to_f(row[off_k + h * dim + i]);
            as[i] = decay[((size_t)t * heads + h) * dim + i];
        }
        if (threadIdx.x < kGlaCols) vs[threadIdx.x] = j0 + threadIdx.x < vdim ? Elem<T>::to_f(row[off_v + h * vdim + j0 + threadIdx.x]) : 0.0f;
        __syncthreads();
        const float v = vs[col];
        float acc = 0.0f;
        for (int i = rg; i < dim; i += kRowGroups) {
            const float sv = fmaf(as[i], S[i * kGlaCols + col], ks[i] * v);
            S[i * kGlaCols + col] = sv;
            acc = fmaf(sv, qs[i], acc);
        }
        part[rg * kGlaCols + col] = acc;
        __syncthreads();
        if (threadIdx.x < kGlaCols && j0 + threadIdx.x < vdim) {
            float r = 0.0f;
#pragma unroll
            for (int g = 0; g < kRowGroups; ++g) r += part[g * kGlaCols + threadIdx.x];
            o[((size_t)t * heads + h) * vdim + j0 + threadIdx.x] = r;
        }
    }
    if (live)
        for (int i = rg; i < dim; i += kRowGroups) slot[(size_t)i * vdim + j0 + col] = S[i * kGlaCols + col];
}

// Register-resident variant (dim <= 32 * RR): the tile of S lives in registers.  A warp owns 8 columns; lane l holds rows l, l + 32, ...
// (RR of them) of those 8 columns, so {decay, k, q} of a row -- one float4 in shared memory -- is loaded once per token and row and used
// for 8 columns, and the 32 lanes read 32 different rows (no broadcast, no bank conflict).  The sum over rows is a butterfly that halves
// the column set at every exchange (4 + 2 + 1 + 1 + 1 shuffles for 8 columns).  Tokens are staged in blocks of TB by four PRODUCER warps
// (global -> fp32 -> shared, two stages) while the four compute warps work on the block before: the global-load latency, which a single
// compute warp per scheduler cannot hide, is off the recurrence's path.  Rows >= dim are zero rows in shared memory: no bounds inside.
constexpr int kGlaWarpCols = 8;
template <typename T, int RR, int TB>
__global__ void __launch_bounds__(256)
gla_recurrent_reg_kernel(const T *__restrict__ proj, int ld, const float *__restrict__ decay, float *__restrict__ state, float *__restrict__ o,
                         const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads,
                         int dim, int vdim, int min_tokens) {
    extern __shared__ __align__(16) float smf[];
    constexpr int DP = 32 * RR;                                  // padded rows
    constexpr int kStage = TB * DP * 4 + TB * kGlaCols;          // floats per stage: {a, k, q, -} [TB][DP] | v [TB][32]
    constexpr int E = TB * DP / 128;                             // staged (token, row) pairs per producer thread
    constexpr int EV = TB * kGlaCols / 128;
    const int j0 = blockIdx.x * kGlaCols, h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp >= 4;                             // warps 4..7 stage the next block of tokens while warps 0..3 compute
    const int c0 = j0 + (warp & 3) * kGlaWarpCols;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (t1 - t0 < min_tokens) return;
    float *slot = state + (((size_t)seq_slot[s] * heads + h) * dim) * vdim;
    const bool fresh = seq_pos0[s] == 0;
    const float qscale = rsqrtf((float)dim);
    const int off_k = heads * dim, off_v = 2 * heads * dim;
    auto fill = [&](int tb, int stage) {  // producer threads: global -> shared, fp32, rows >= dim and tokens >= t1 as zeros
        float4 *akq = reinterpret_cast<float4 *>(smf + stage * kStage);
        float *vs = smf + stage * kStage + TB * DP * 4;
        const int ptid = threadIdx.x - 128;
        // every load first (addresses clamped into range so that none is conditional and all are in flight together), then the stores
        float ra[E], rk[E], rq[E], rv[EV];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int idx = ptid + e * 128;
            const int tt = idx / DP, i = min(idx % DP, dim - 1), t = min(tb + tt, t1 - 1);
            const T *row = proj + (size_t)t * ld;
            ra[e] = decay[((size_t)t * heads + h) * dim + i];
            rk[e] = Elem<T>::to_f(row[off_k + h * dim + i]);
            rq[e] = Elem<T>::to_f(row[h * dim + i]);
        }
#pragma unroll
        for (int e = 0; e < EV; ++e) {
            const int idx = ptid + e * 128;
            const int tt = idx / kGlaCols, c = min(j0 + idx % kGlaCols, vdim - 1), t = min(tb + tt, t1 - 1);
            rv[e] = Elem<T>::to_f(proj[(size_t)t * ld + off_v + h * vdim + c]);
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int idx = ptid + e * 128;
            const bool live = tb + idx / DP < t1 && idx % DP < dim;
            akq[idx] = live ? make_float4(ra[e], rk[e], rq[e] * qscale, 0.0f) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int e = 0; e < EV; ++e) {
            const int idx = ptid + e * 128;
            vs[idx] = (tb + idx / kGlaCols < t1 && j0 + idx % kGlaCols < vdim) ? rv[e] : 0.0f;
        }
    };
    float S[RR][kGlaWarpCols];
    if (!producer) {
#pragma unroll
        for (int r = 0; r < RR; ++r)
#pragma unroll
            for (int c = 0; c < kGlaWarpCols; ++c) {
                const int i = lane + 32 * r;
                S[r][c] = (!fresh && i < dim && c0 + c < vdim) ? slot[(size_t)i * vdim + c0 + c] : 0.0f;
            }
    } else {
        fill(t0, 0);
    }
    __syncthreads();
    int stage = 0;
    for (int tb = t0; tb < t1; tb += TB, stage ^= 1) {
        if (producer) {
            if (tb + TB < t1) fill(tb + TB, stage ^ 1);
        } else {
            const float4 *akq = reinterpret_cast<const float4 *>(smf + stage * kStage);
            const float *vs = smf + stage * kStage + TB * DP * 4;
            const int nt = min(TB, t1 - tb);
            // one token's update of S and its 8 per-lane partial outputs
            auto advance = [&](int tt, float *acc) {
                const float4 v0 = *reinterpret_cast<const float4 *>(vs + tt * kGlaCols + warp * kGlaWarpCols);
                const float4 v1 = *reinterpret_cast<const float4 *>(vs + tt * kGlaCols + warp * kGlaWarpCols + 4);
                const float v[kGlaWarpCols] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                for (int c = 0; c < kGlaWarpCols; ++c) acc[c] = 0.0f;
#pragma unroll
                for (int r = 0; r < RR; ++r) {
                    const float4 x = akq[tt * DP + lane + 32 * r];
#pragma unroll
                    for (int c = 0; c < kGlaWarpCols; ++c) {
                        S[r][c] = fmaf(x.x, S[r][c], x.y * v[c]);
                        acc[c] = fmaf(S[r][c], x.z, acc[c]);
                    }
                }
            };
            // butterfly over the 32 lanes, halving the columns a lane is responsible for: 8 -> 4 -> 2 -> 1, then two plain steps
            auto reduce = [&](const float *acc) -> float {
                float a4[4], a2[2], a1;
                {
                    const bool up = lane & 16;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float give = up ? acc[c] : acc[c + 4], keep = up ? acc[c + 4] : acc[c];
                        a4[c] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
                    }
                }
                {
                    const bool up = lane & 8;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const float give = up ? a4[c] : a4[c + 2], keep = up ? a4[c + 2] : a4[c];
                        a2[c] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
                    }
                }
                {
                    const bool up = lane & 4;
                    const float give = up ? a2[0] : a2[1], keep = up ? a2[1] : a2[0];
                    a1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
                }
                a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
                a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
                return a1;  // every lane of a group of four holds column ((l >> 4) & 1) * 4 + ((l >> 3) & 1) * 2 + ((l >> 2) & 1)
            };
            const int ocol = c0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
            // tokens in groups: the updates of S are a short serial chain, the reductions are independent of one
            // another and sit in one straight-line block, so their shuffle latencies overlap instead of adding up per token
            int tt = 0;
            constexpr int GS = 8;  // tokens per group
            for (; tt + GS <= nt; tt += GS) {
                float accg[GS][kGlaWarpCols];
#pragma unroll
                for (int u = 0; u < GS; ++u) advance(tt + u, accg[u]);
                float rg[GS];
#pragma unroll
                for (int u = 0; u < GS; ++u) rg[u] = reduce(accg[u]);
                // lane l of a group of four stores tokens (l & 3), (l & 3) + 4: no branch per token
                const int u = lane & 3;
#pragma unroll
                for (int half = 0; half < GS / 4; ++half) {
                    const float val = u == 0 ? rg[4 * half] : (u == 1 ? rg[4 * half + 1] : (u == 2 ? rg[4 * half + 2] : rg[4 * half + 3]));
                    if (ocol < vdim) o[((size_t)(tb + tt + 4 * half + u) * heads + h) * vdim + ocol] = val;
                }
            }
            for (; tt < nt; ++tt) {
                float acc[kGlaWarpCols];
                advance(tt, acc);
                const float val = reduce(acc);
                if ((lane & 3) == 0 && ocol < vdim) o[((size_t)(tb + tt) * heads + h) * vdim + ocol] = val;
            }
        }
        __syncthreads();  // the next stage is filled and this one consumed
    }
    if (producer) return;
#pragma unroll
    for (int r = 0; r < RR; ++r)
#pragma unroll
        for (int c = 0; c < kGlaWarpCols; ++c) {
            const int i = lane + 32 * r;
            if (i < dim && c0 + c < vdim) slot[(size_t)i * vdim + c0 + c] = S[r][c];
        }
}

// One-token portions (decoding): the step is a single pass over the sequence's state, so the kernel is laid out for the memory system
// instead of the token loop.  A CTA owns kStepCols columns of one (sequence, head); a thread owns four consecutive columns (one 16-byte
// piece of a state row) and every 16th row, the loads of a thread's rows are issued together, and the 16 row groups' partial outputs meet
// in shared memory.  Sequences with more than one token leave at once (the token-loop kernel serves them) and vice versa.
constexpr int kStepCols = 64;
constexpr int kStepRowGroups = 16;
constexpr int kStepUnroll = 8;
template <typename T>
__global__ void __launch_bounds__(256)
gla_step_kernel(const T *__restrict__ proj, int ld, const float *__restrict__ decay, float *__restrict__ state, float *__restrict__ o,
                const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads, int dim,
                int vdim) {
    extern __shared__ __align__(16) float smf[];  // {a, k, q, -}[dim] | part[kStepRowGroups][kStepCols]
    const int s = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * kStepCols;
    const int t = seq_start[s];
    if (seq_start[s + 1] - t != 1) return;
    float4 *akq = reinterpret_cast<float4 *>(smf);
    float *part = smf + 4 * (size_t)dim;
    const T *row = proj + (size_t)t * ld;
    const float qscale = rsqrtf((float)dim);
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        akq[i] = make_float4(decay[((size_t)t * heads + h) * dim + i], Elem<T>::to_f(row[heads * dim + h * dim + i]),
                             Elem<T>::to_f(row[h * dim + i]) * qscale, 0.0f);
    const int cg = threadIdx.x % (kStepCols / 4), rg = threadIdx.x / (kStepCols / 4);
    const int c = j0 + 4 * cg;
    const bool live = c < vdim;  // vdim is a multiple of 4 here
    const bool fresh = seq_pos0[s] == 0;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = Elem<T>::to_f(row[2 * heads * dim + h * vdim + c + e]);
    }
    float *slot = state + (((size_t)seq_slot[s] * heads + h) * dim) * vdim + c;
    __syncthreads();
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
        for (int i0 = rg; i0 < dim; i0 += kStepRowGroups * kStepUnroll) {
            float4 sv[kStepUnroll];
#pragma unroll
            for (int u = 0; u < kStepUnroll; ++u) {
                const int i = i0 + u * kStepRowGroups;
                sv[u] = (!fresh && i < dim) ? *reinterpret_cast<const float4 *>(slot + (size_t)i * vdim) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < kStepUnroll; ++u) {
                const int i = i0 + u * kStepRowGroups;
                if (i < dim) {
                    const float4 x = akq[i];
                    float4 n;
                    n.x = fmaf(x.x, sv[u].x, x.y * v[0]);
                    n.y = fmaf(x.x, sv[u].y, x.y * v[1]);
                    n.z = fmaf(x.x, sv[u].z, x.y * v[2]);
                    n.w = fmaf(x.x, sv[u].w, x.y * v[3]);
                    *reinterpret_cast<float4 *>(slot + (size_t)i * vdim) = n;
                    acc[0] = fmaf(n.x, x.z, acc[0]);
                    acc[1] = fmaf(n.y, x.z, acc[1]);
                    acc[2] = fmaf(n.z, x.z, acc[2]);
                    acc[3] = fmaf(n.w, x.z, acc[3]);
                }
            }
        }
    }
    *reinterpret_cast<float4 *>(part + rg * kStepCols + 4 * cg) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (threadIdx.x < kStepCols && j0 + threadIdx.x < vdim) {
        float r = 0.0f;
#pragma unroll
        for (int g = 0; g < kStepRowGroups; ++g) r += part[g * kStepCols + threadIdx.x];
        o[((size_t)t * heads + h) * vdim + j0 + threadIdx.x] = r;
    }
}

template <typename T, int RR, int TB>
static void launch_gla_reg(const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start, const int *seq_pos0,
                           const int *seq_slot, dim3 grid, int heads, int dim, int vdim, int min_tokens, cudaStream_t st) {
    const size_t smem = 2 * ((size_t)TB * 32 * RR * 4 + (size_t)TB * kGlaCols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gla_recurrent_reg_kernel<T, RR, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gla_recurrent_reg_kernel<T, RR, TB><<<grid, 256, smem, st>>>((const T *)proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, heads, dim, vdim, min_tokens);
}

template <typename T>
__global__ void __launch_bounds__(128)
gla_output_kernel(const float *__restrict__ o, const float *__restrict__ w, float eps, const T *__restrict__ gate_in, int gate_ld,
                  T *__restrict__ out, int heads, int vdim) {
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y;
    const float *orow = o + ((size_t)t * heads + h) * vdim;
    constexpr int V = Elem<T>::kVec;
    const T *grow = gate_in + (size_t)t * gate_ld + h * vdim;
    T *out_row = out + ((size_t)t * heads + h) * vdim;
    // 16-byte pieces when every row starts on a 16-byte boundary
    const bool vec = vdim % V == 0 && gate_ld % V == 0 && vdim <= (int)blockDim.x * V &&
                     ((reinterpret_cast<size_t>(o) | reinterpret_cast<size_t>(w) | reinterpret_cast<size_t>(gate_in) | reinterpret_cast<size_t>(out)) & 15) == 0;
    float ss = 0.0f;
    if (vec) {
        float ov[V], gz[V];
        const int j = threadIdx.x * V;  // the launcher gives a row's pieces one thread each
        if (j < vdim) {
#pragma unroll
            for (int e = 0; e < V; e += 4) {
                const float4 a = *reinterpret_cast<const float4 *>(orow + j + e);
                ov[e] = a.x, ov[e + 1] = a.y, ov[e + 2] = a.z, ov[e + 3] = a.w;
            }
            unpack16<T>(ld_v4(grow + j), gz);
#pragma unroll
            for (int e = 0; e < V; ++e) ss = fmaf(ov[e], ov[e], ss);
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)vdim + eps);
        if (j < vdim) {
            float y[V];
#pragma unroll
            for (int e = 0; e < V; ++e) y[e] = ov[e] * inv * w[j + e] * (gz[e] / (1.0f + expf(-gz[e])));
            st_v4(out_row + j, pack16<T>(y));
        }
        return;
    }
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) ss = fmaf(orow[j], orow[j], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
        const float z = Elem<T>::to_f(grow[j]);
        const float y = orow[j] * inv * w[j] * (z / (1.0f + expf(-z)));
        out_row[j] = Elem<T>::from_f(y);
    }
}

int launch_gla_decay(int dtype, const void *proj, int ld, int col0, const void *w_decay, const float *bias, float tau, float *decay,
                     int tokens, int rank, int channels, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        // few token blocks (decoding): the channels are spread over CTAs as well
        const int nb = (tokens + kDecayTokens - 1) / kDecayTokens;
        const int cb = nb >= 64 ? 1 : (channels + 255) / 256;
        gla_decay_kernel<T><<<dim3(nb, cb), 256, (size_t)kDecayTokens * rank * sizeof(float), st>>>(
            (const T *)proj, ld, col0, (const T *)w_decay, bias, 1.0f / tau, decay, tokens, rank, channels);
    });
    return cuda_status("gla_decay launch");
}

int launch_gla_recurrent(int dtype, const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start,
                         const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st, int kinds) {
    if (n_seqs == 0) return B200_OK;
    // one-token portions take the step kernel (16-byte pieces of state rows: vdim a multiple of 4); the token-loop kernels then skip them
    const bool step = (kinds & kGlaOneToken) && vdim % 4 == 0 && (reinterpret_cast<size_t>(state) & 15) == 0 &&
                      (4 * (size_t)dim + kStepRowGroups * kStepCols) * sizeof(float) <= 200 * 1024;
    if (step) {
        const size_t smem_step = (4 * (size_t)dim + kStepRowGroups * kStepCols) * sizeof(float);
        const dim3 grid_step((vdim + kStepCols - 1) / kStepCols, heads, n_seqs);
        B200_DISPATCH_DTYPE(dtype, {
            if (smem_step > 48 * 1024) cudaFuncSetAttribute(gla_step_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_step);
            gla_step_kernel<T><<<grid_step, 256, smem_step, st>>>((const T *)proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, heads, dim, vdim);
        });
        if (!(kinds & kGlaManyTokens)) return cuda_status("gla_step launch");
    }
    const int min_tokens = step ? 2 : 1;
    const size_t smem = ((size_t)dim * kGlaCols + 3 * (size_t)dim + kGlaCols + (kGlaThreads / kGlaCols) * kGlaCols) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("gla_recurrent: key size %d does not fit the shared-memory state tile", dim);
        return B200_ERR_UNSUPPORTED;
    }
    const dim3 grid((vdim + kGlaCols - 1) / kGlaCols, heads, n_seqs);
    if (dim <= 256) {
        B200_DISPATCH_DTYPE(dtype, {
            if (dim <= 32) launch_gla_reg<T, 1, 16>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, min_tokens, st);
            else if (dim <= 64) launch_gla_reg<T, 2, 16>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, min_tokens, st);
            else if (dim <= 128) launch_gla_reg<T, 4, 16>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, min_tokens, st);
            else launch_gla_reg<T, 8, 8>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, min_tokens, st);
        });
        return cuda_status("gla_recurrent launch");
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(gla_recurrent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gla_recurrent_kernel<T><<<grid, kGlaThreads, smem, st>>>((const T *)proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, heads, dim,
                                                                  vdim, min_tokens);
    });
    return cuda_status("gla_recurrent launch");
}

int launch_gla_output(int dtype, const float *o, const float *w, float eps, const void *gate_in, int gate_ld, void *out, int tokens,
                      int heads, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        constexpr int V = Elem<T>::kVec;
        // rows that go in 16-byte pieces need one thread per piece; others keep 128 threads striding the row
        const int threads = (vdim % V == 0 && vdim / V <= 128) ? std::max(32, (vdim / V + 31) / 32 * 32) : 128;
        gla_output_kernel<T><<<dim3(tokens, heads), threads, 0, st>>>(o, w, eps, (const T *)gate_in, gate_ld, (T *)out, heads, vdim);
    });
    return cuda_status("gla_output launch");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gla_recurrent(const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start,
                                  const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, int dtype,
                                  b200_stream_t stream) {
    B200_REQUIRE(proj && decay && state && o && seq_start && seq_pos0 && seq_slot, "gla_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0 && ld >= 2 * heads * dim + heads * vdim, "gla_recurrent: bad shape");
    return launch_gla_recurrent(dtype, proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, n_seqs, heads, dim, vdim, as_stream(stream));
}
