// gla.cu -- gated linear attention (a linear-attention recurrence with a learned decay per key channel):
//     a_t = sigmoid(z_t)^(1/tau),  z_t = W2 (W1 h_t) + b           (heads x dim channels, fp32 from the low-rank projection on)
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T                           (per head, S is dim x vdim, fp32)
//     o_t = S_t^T (q_t / sqrt(dim))
//     y_t = rmsnorm_vdim(o_t) * w * silu(gate_t)                    (per head; w shared by the heads)
// The state of a sequence lives in a slot of a pool ([slots, heads, dim, vdim] fp32) between calls; a portion that starts at position 0
// starts from zero.  Columns of S are independent of one another, so a head is cut into column tiles, one CTA each: the grid is
// (vdim tiles, heads, sequences), the token loop is serial inside a CTA, the tile of S stays in shared memory for the whole portion.
// Decoding is the same kernel with one token per sequence.
#include "hybrid_ops.cuh"

namespace b200 {

constexpr int kGlaCols = 32;     // columns of S per CTA
constexpr int kGlaThreads = 256; // 8 row groups x 32 columns

template <typename T>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const T *__restrict__ proj, int ld, int col0, const T *__restrict__ w, const float *__restrict__ bias, float inv_tau,
                 float *__restrict__ decay, int rank, int channels) {
    extern __shared__ float lo[];  // the token's low-rank vector
    const int t = blockIdx.x;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) lo[r] = Elem<T>::to_f(proj[(size_t)t * ld + col0 + r]);
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float z = bias ? bias[c] : 0.0f;
        const T *wr = w + (size_t)c * rank;
        for (int r = 0; r < rank; ++r) z = fmaf(Elem<T>::to_f(wr[r]), lo[r], z);
        // log sigmoid(z) = min(z, 0) - log1p(exp(-|z|));  a = exp(log sigmoid(z) / tau)
        const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
        decay[(size_t)t * channels + c] = expf(ls * inv_tau);
    }
}

// Shared memory: S[dim][kGlaCols] | q[dim] | k[dim] | a[dim] | v[kGlaCols] | part[8][kGlaCols]
template <typename T>
__global__ void __launch_bounds__(kGlaThreads)
gla_recurrent_kernel(const T *__restrict__ proj, int ld, const float *__restrict__ decay, float *__restrict__ state, float *__restrict__ o,
                     const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads,
                     int dim, int vdim) {
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
    if (t1 <= t0) return;
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

// Register-resident variant (dim <= 4 * R): the tile of S lives in registers, R rows per thread.  A warp owns 8 columns; its lanes are
// 8 columns x 4 row groups (rows rg, rg + 4, ...), so the sum over rows ends with two shuffles and no barrier.  Tokens are staged in
// blocks of TB: {decay, k, q} of a row as one float4 in shared memory (one 16-byte broadcast load per row and token), the next block's
// global loads are issued before the current block is computed.  One barrier pair per TB tokens.
template <typename T, int R, int TB>
__global__ void __launch_bounds__(128)
gla_recurrent_reg_kernel(const T *__restrict__ proj, int ld, const float *__restrict__ decay, float *__restrict__ state, float *__restrict__ o,
                         const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads,
                         int dim, int vdim) {
    extern __shared__ __align__(16) float smf[];
    float4 *akq = reinterpret_cast<float4 *>(smf);              // [TB][dim]
    float *vs = smf + (size_t)TB * dim * 4;                      // [TB][32]
    constexpr int E = TB * R / 32;                               // staged (row, token) pairs per thread
    const int j0 = blockIdx.x * kGlaCols, h = blockIdx.y, s = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, cg = lane & 7, rg = lane >> 3;
    const int col = j0 + warp * 8 + cg;
    const bool live = col < vdim;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    if (t1 <= t0) return;
    float *slot = state + (((size_t)seq_slot[s] * heads + h) * dim) * vdim;
    const bool fresh = seq_pos0[s] == 0;
    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = rg + 4 * r;
        S[r] = (!fresh && live && i < dim) ? slot[(size_t)i * vdim + col] : 0.0f;
    }
    const float qscale = rsqrtf((float)dim);
    const int off_k = heads * dim, off_v = 2 * heads * dim;
    constexpr int EV = TB * kGlaCols / 128;                      // staged values per thread
    float pa[E], pk[E], pq[E], pv[EV];
    auto fetch = [&](int tb) {  // global -> registers
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int idx = threadIdx.x + e * 128;
            const int tt = idx / dim, i = idx - tt * dim, t = tb + tt;
            if (tt < TB && t < t1) {
                const T *row = proj + (size_t)t * ld;
                pa[e] = decay[((size_t)t * heads + h) * dim + i];
                pk[e] = Elem<T>::to_f(row[off_k + h * dim + i]);
                pq[e] = Elem<T>::to_f(row[h * dim + i]) * qscale;
            }
        }
#pragma unroll
        for (int e = 0; e < EV; ++e) {
            const int idx = threadIdx.x + e * 128;
            const int tt = idx / kGlaCols, c = idx - tt * kGlaCols, t = tb + tt;
            pv[e] = (t < t1 && j0 + c < vdim) ? Elem<T>::to_f(proj[(size_t)t * ld + off_v + h * vdim + j0 + c]) : 0.0f;
        }
    };
    auto stash = [&](int tb) {  // registers -> shared
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int idx = threadIdx.x + e * 128;
            const int tt = idx / dim, i = idx - tt * dim;
            if (tt < TB && tb + tt < t1) akq[tt * dim + i] = make_float4(pa[e], pk[e], pq[e], 0.0f);
        }
#pragma unroll
        for (int e = 0; e < EV; ++e) vs[threadIdx.x + e * 128] = pv[e];
    };
    fetch(t0);
    for (int tb = t0; tb < t1; tb += TB) {
        __syncthreads();  // the previous block has been consumed
        stash(tb);
        __syncthreads();
        if (tb + TB < t1) fetch(tb + TB);
        const int nt = min(TB, t1 - tb);
        for (int tt = 0; tt < nt; ++tt) {
            const float v = vs[tt * kGlaCols + warp * 8 + cg];
            const float4 *row = akq + tt * dim + rg;
            float acc = 0.0f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (rg + 4 * r < dim) {
                    const float4 x = row[4 * r];
                    S[r] = fmaf(x.x, S[r], x.y * v);
                    acc = fmaf(S[r], x.z, acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (rg == 0 && live) o[((size_t)(tb + tt) * heads + h) * vdim + col] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = rg + 4 * r;
            if (i < dim) slot[(size_t)i * vdim + col] = S[r];
        }
    }
}

template <typename T, int R, int TB>
static void launch_gla_reg(const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start, const int *seq_pos0,
                           const int *seq_slot, dim3 grid, int heads, int dim, int vdim, cudaStream_t st) {
    const size_t smem = ((size_t)TB * dim * 4 + (size_t)TB * kGlaCols) * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(gla_recurrent_reg_kernel<T, R, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gla_recurrent_reg_kernel<T, R, TB><<<grid, 128, smem, st>>>((const T *)proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, heads, dim, vdim);
}

template <typename T>
__global__ void __launch_bounds__(128)
gla_output_kernel(const float *__restrict__ o, const float *__restrict__ w, float eps, const T *__restrict__ gate_in, int gate_ld,
                  T *__restrict__ out, int heads, int vdim) {
    __shared__ float red[33];
    const int t = blockIdx.x, h = blockIdx.y;
    const float *orow = o + ((size_t)t * heads + h) * vdim;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) ss = fmaf(orow[j], orow[j], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = threadIdx.x; j < vdim; j += blockDim.x) {
        const float z = Elem<T>::to_f(gate_in[(size_t)t * gate_ld + h * vdim + j]);
        const float y = orow[j] * inv * w[j] * (z / (1.0f + expf(-z)));
        out[((size_t)t * heads + h) * vdim + j] = Elem<T>::from_f(y);
    }
}

int launch_gla_decay(int dtype, const void *proj, int ld, int col0, const void *w_decay, const float *bias, float tau, float *decay,
                     int tokens, int rank, int channels, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        gla_decay_kernel<T><<<tokens, 256, (size_t)rank * sizeof(float), st>>>((const T *)proj, ld, col0, (const T *)w_decay, bias, 1.0f / tau,
                                                                                decay, rank, channels);
    });
    return cuda_status("gla_decay launch");
}

int launch_gla_recurrent(int dtype, const void *proj, int ld, const float *decay, float *state, float *o, const int *seq_start,
                         const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st) {
    if (n_seqs == 0) return B200_OK;
    const size_t smem = ((size_t)dim * kGlaCols + 3 * (size_t)dim + kGlaCols + (kGlaThreads / kGlaCols) * kGlaCols) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("gla_recurrent: key size %d does not fit the shared-memory state tile", dim);
        return B200_ERR_UNSUPPORTED;
    }
    const dim3 grid((vdim + kGlaCols - 1) / kGlaCols, heads, n_seqs);
    if (dim <= 256) {
        B200_DISPATCH_DTYPE(dtype, {
            if (dim <= 64) launch_gla_reg<T, 16, 16>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, st);
            else if (dim <= 128) launch_gla_reg<T, 32, 16>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, st);
            else launch_gla_reg<T, 64, 8>(proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, grid, heads, dim, vdim, st);
        });
        return cuda_status("gla_recurrent launch");
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(gla_recurrent_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gla_recurrent_kernel<T><<<grid, kGlaThreads, smem, st>>>((const T *)proj, ld, decay, state, o, seq_start, seq_pos0, seq_slot, heads, dim,
                                                                  vdim);
    });
    return cuda_status("gla_recurrent launch");
}

int launch_gla_output(int dtype, const float *o, const float *w, float eps, const void *gate_in, int gate_ld, void *out, int tokens,
                      int heads, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        gla_output_kernel<T><<<dim3(tokens, heads), 128, 0, st>>>(o, w, eps, (const T *)gate_in, gate_ld, (T *)out, heads, vdim);
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
