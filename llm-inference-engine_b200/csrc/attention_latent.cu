// attention_latent.cu -- latent attention over a paged pool, for ragged mixed batches.
//
// Every position caches ONE row shared by all heads: [c (kv_rank) | kr (rot_dim)], c the RMS-normed low-rank projection of the layer's
// input and kr a rotated key part.  Per head the key would be [W_uk,h c | kr] and the value W_uv,h c; instead of expanding the cached rows
// the query is moved into the latent space (the "absorbed" form):
//     score_h(i, j) = scale * ( (W_uk,h^T qn_h(i)) . c(j) + qr_h(i) . kr(j) ),      out_h(i) = W_uv,h ( sum_j p_h(i, j) c(j) )
// so attention is multi-query attention over rows of kv_rank + rot_dim with the first kv_rank columns doubling as values, and the two
// per-head products are grouped GEMMs over the heads (rows grouped head by head: [heads, t_pad, *], t_pad a whole number of row tiles).
// The same form serves prompt portions and single decoded tokens, so a position's logits do not depend on how its prompt was cut.
//   * latent_prep_kernel: splits the fused projection: qn (un-rotated query part) regrouped by head, qr rotated, and -- for a layer with a
//     cache of its own -- the latent row normed (fp32) and the key part rotated, appended to the pool.  Angles are formed in fp64.
//   * latent_attn_kernel: one CTA per (token, head): sliding window (i sees j with 0 <= i - j < window), softmax in fp32 with a per-head
//     sink logit in the denominator, weighted sum of the latent rows.
//   * latent_attn_mma_kernel: the tensor-core form for 16-bit engines: one CTA per tile of <= 64 query rows that share their keys (64
//     consecutive tokens of one sequence x one head), key tiles of one page through a cp.async ring, the value operand read from the
//     key tile's own first columns.
//   * latent_gate_kernel: back to token-major rows, times sigmoid(gate).
#include "hybrid_ops.cuh"

#include <algorithm>

namespace b200 {

namespace {
constexpr int kPageL = B200_KV_PAGE_SIZE;
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T *__restrict__ proj, int ld, int q_col, int kv_col, T *__restrict__ qn, T *__restrict__ qr, T *__restrict__ pool,
                   const float *__restrict__ kv_norm, float eps, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                   const int *__restrict__ block_table, int mpps, int t_pad, int heads, int dim, int rot_dim, int kv_rank, int rot_dims,
                   float rot_base) {
    extern __shared__ float cs[];  // cos[half] | sin[half]
    __shared__ float red[33];
    const int t = blockIdx.x, half = rot_dims / 2;
    const int pos = tok_pos[t];
    float *cosv = cs, *sinv = cs + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const double f = exp2(-2.0 * (double)i / (double)rot_dims * log2((double)rot_base));
        double s, c;
        sincos((double)pos * f, &s, &c);
        cosv[i] = (float)c, sinv[i] = (float)s;
    }
    __syncthreads();
    const T *row = proj + (size_t)t * ld;
    // r-th element of a rotated vector that starts at `v`
    auto rotated = [&](const T *v, int r) -> float {
        const float self = Elem<T>::to_f(v[r]);
        if (r < half) return self * cosv[r] - Elem<T>::to_f(v[r + half]) * sinv[r];
        if (r < rot_dims) return self * cosv[r - half] + Elem<T>::to_f(v[r - half]) * sinv[r - half];
        return self;
    };
    const int per = dim + rot_dim;
    for (int idx = threadIdx.x; idx < heads * per; idx += blockDim.x) {
        const int h = idx / per, c = idx - h * per;
        const T *qh = row + q_col + (size_t)h * per;
        if (c < dim) qn[((size_t)h * t_pad + t) * dim + c] = qh[c];
        else qr[((size_t)t * heads + h) * rot_dim + (c - dim)] = Elem<T>::from_f(rotated(qh + dim, c - dim));
    }
    if (kv_col < 0) return;  // this layer reads another layer's rows
    const T *kv = row + kv_col;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const float v = Elem<T>::to_f(kv[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)kv_rank + eps);
    const int page = block_table[(size_t)tok_seq[t] * mpps + pos / kPageL];
    if (page < 0) return;  // no page held: nothing is written (the host refuses such a batch)
    T *dst = pool + ((size_t)page * kPageL + (pos % kPageL)) * (kv_rank + rot_dim);
    for (int c = threadIdx.x; c < kv_rank + rot_dim; c += blockDim.x)
        dst[c] = Elem<T>::from_f(c < kv_rank ? Elem<T>::to_f(kv[c]) * inv * kv_norm[c] : rotated(kv + kv_rank, c - kv_rank));
}

// One CTA per (token, head).  Shared memory: q[kv_rank + rot_dim] | scores[max_keys] | partial sums | red[33].
template <typename T>
__global__ void __launch_bounds__(256)
latent_attn_kernel(const T *__restrict__ ql, const T *__restrict__ qr, const T *__restrict__ pool, const float *__restrict__ sink,
                   T *__restrict__ ol, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ block_table,
                   int mpps, int t_pad, int heads, int kv_rank, int rot_dim, float scale, int window, int max_keys, int part_floats,
                   const int *__restrict__ tok_list) {
    extern __shared__ __align__(16) float sm[];
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    const int dk = kv_rank + rot_dim;
    const int pos = tok_pos[t];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int nkeys = pos - first + 1;
    float *qs = sm;
    float *sc = qs + (dk + 3) / 4 * 4;
    float *part = sc + (max_keys + 3) / 4 * 4;
    float *red = part + part_floats;
    const int *bt = block_table + (size_t)tok_seq[t] * mpps;
    for (int c = threadIdx.x; c < dk; c += blockDim.x)
        qs[c] = Elem<T>::to_f(c < kv_rank ? ql[((size_t)h * t_pad + t) * kv_rank + c] : qr[((size_t)t * heads + h) * rot_dim + (c - kv_rank)]);
    __syncthreads();

    constexpr int V = Elem<T>::kVec;
    const bool vec = dk % V == 0 && kv_rank % V == 0 && (reinterpret_cast<size_t>(pool) & 15) == 0;
    float mx = sink ? sink[h] : -INFINITY;
    if (vec) {
        // eight adjacent lanes share a key row, each takes every eighth 16-byte piece
        const int sub = threadIdx.x & 7, kslot = threadIdx.x >> 3, nslots = blockDim.x >> 3, pieces = dk / V;
        for (int j0 = 0; j0 < nkeys; j0 += nslots) {  // warp-uniform trip count: the shuffles below take every lane
            const int j = j0 + kslot;
            const int p = first + min(j, nkeys - 1);
            const T *kr = pool + ((size_t)bt[p / kPageL] * kPageL + (p % kPageL)) * dk;
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
            for (int pc = sub; pc < pieces; pc += 8) {
                float f[V];
                unpack16<T>(ld_v4(kr + pc * V), f);
                const float *qp = qs + pc * V;
#pragma unroll
                for (int i = 0; i < V; i += 2) {
                    a0 = fmaf(qp[i], f[i], a0);
                    a1 = fmaf(qp[i + 1], f[i + 1], a1);
                }
            }
            float acc = a0 + a1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc *= scale;
            if (j < nkeys) {
                if (sub == 0) sc[j] = acc;
                mx = fmaxf(mx, acc);
            }
        }
    } else {
        for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
            const int p = first + j;
            const T *kr = pool + ((size_t)bt[p / kPageL] * kPageL + (p % kPageL)) * dk;
            float acc = 0.0f;
            for (int c = 0; c < dk; ++c) acc = fmaf(qs[c], Elem<T>::to_f(kr[c]), acc);
            acc *= scale;
            sc[j] = acc;
            mx = fmaxf(mx, acc);
        }
    }
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = block_sum(sum, red);  // (its barriers also publish sc[])
    if (sink) sum += expf(sink[h] - mx);  // the sink: a logit with no key and no value, counted once
    const float inv = 1.0f / sum;

    // ---- weighted sum of the latent rows (the first kv_rank columns of the same pool rows)
    T *orow = ol + ((size_t)h * t_pad + t) * kv_rank;
    const int tpr = kv_rank / V;  // threads per row when a thread takes one 16-byte piece
    if (vec && tpr <= (int)blockDim.x) {
        const int groups = (int)blockDim.x / tpr, kg = threadIdx.x / tpr, c0 = (threadIdx.x - kg * tpr) * V;
        if (kg < groups) {
            float acc[V];
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.0f;
#pragma unroll 4
            for (int j = kg; j < nkeys; j += groups) {
                const int p = first + j;
                float f[V];
                unpack16<T>(ld_v4(pool + ((size_t)bt[p / kPageL] * kPageL + (p % kPageL)) * dk + c0), f);
                const float w = sc[j];
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(w, f[i], acc[i]);
            }
#pragma unroll
            for (int i = 0; i < V; ++i) part[kg * kv_rank + c0 + i] = acc[i];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
            float a = 0.0f;
            for (int k2 = 0; k2 < groups; ++k2) a += part[k2 * kv_rank + c];
            orow[c] = Elem<T>::from_f(a * inv);
        }
        return;
    }
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < nkeys; ++j) {
            const int p = first + j;
            acc = fmaf(sc[j], Elem<T>::to_f(pool[((size_t)bt[p / kPageL] * kPageL + (p % kPageL)) * dk + c]), acc);
        }
        orow[c] = Elem<T>::from_f(acc * inv);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
latent_gate_kernel(const T *__restrict__ ov, const T *__restrict__ gate_in, int gate_ld, T *__restrict__ out, int t_pad, int heads, int vdim) {
    const int t = blockIdx.x;
    for (int idx = threadIdx.x; idx < heads * vdim; idx += blockDim.x) {
        const int h = idx / vdim, c = idx - h * vdim;
        const float z = Elem<T>::to_f(gate_in[(size_t)t * gate_ld + idx]);
        out[(size_t)t * heads * vdim + idx] = Elem<T>::from_f(Elem<T>::to_f(ov[((size_t)h * t_pad + t) * vdim + c]) / (1.0f + expf(-z)));
    }
}

int launch_latent_prep(int dtype, const void *proj, int ld, int q_col, int kv_col, void *qn, void *qr, void *pool, const float *kv_norm,
                       float eps, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps, int tokens, int t_pad, int heads,
                       int dim, int rot_dim, int kv_rank, int rot_dims, float rot_base, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const size_t smem = (size_t)std::max(rot_dims, 2) * sizeof(float);
    B200_DISPATCH_DTYPE(dtype, {
        latent_prep_kernel<T><<<tokens, 128, smem, st>>>((const T *)proj, ld, q_col, kv_col, (T *)qn, (T *)qr, (T *)pool, kv_norm, eps, tok_seq,
                                                        tok_pos, block_table, mpps, t_pad, heads, dim, rot_dim, kv_rank, rot_dims, rot_base);
    });
    return cuda_status("latent_prep launch");
}

int launch_latent_attention(int dtype, const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tok_seq,
                            const int *tok_pos, const int *block_table, int mpps, int tokens, int t_pad, int heads, int kv_rank, int rot_dim,
                            float scale, int window, int max_keys, cudaStream_t st, const int *tok_list) {
    if (tokens == 0) return B200_OK;
    const int threads = max_keys >= 128 ? 256 : 128;
    const int vlen = dtype == B200_F32 ? 4 : 8;
    const int tpr = std::max(1, kv_rank / vlen);
    const int groups = std::max(1, threads / tpr);
    const size_t part = (size_t)groups * kv_rank;
    const size_t smem = ((size_t)(kv_rank + rot_dim + 3) / 4 * 4 + (size_t)(max_keys + 3) / 4 * 4 + part + 33) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("latent_attention: %d keys x rank %d do not fit the shared-memory score buffer", max_keys, kv_rank);
        return B200_ERR_UNSUPPORTED;
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        latent_attn_kernel<T><<<dim3(tokens, heads), threads, smem, st>>>((const T *)ql, (const T *)qr, (const T *)pool, sink, (T *)ol, tok_seq,
                                                                           tok_pos, block_table, mpps, t_pad, heads, kv_rank, rot_dim, scale,
                                                                           window, max_keys, (int)part, tok_list);
    });
    return cuda_status("latent_attention launch");
}

int launch_latent_gate(int dtype, const void *ov, const void *gate_in, int gate_ld, void *out, int tokens, int t_pad, int heads, int vdim,
                       cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        latent_gate_kernel<T><<<tokens, 256, 0, st>>>((const T *)ov, (const T *)gate_in, gate_ld, (T *)out, t_pad, heads, vdim);
    });
    return cuda_status("latent_gate launch");
}

}  // namespace b200
