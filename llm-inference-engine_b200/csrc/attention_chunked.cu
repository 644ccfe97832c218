// attention_chunked.cu -- softmax attention without rotation over a paged key/value pool, for ragged mixed batches:
//   * attn_qk_norm_cache_kernel: RMS norm over the WHOLE q projection and the WHOLE k projection (all heads at once), q to a dense
//     buffer, normed k to the K pool, k as projected to the V pool (the values of this mixer are its un-normed keys);
//   * chunked_attn_kernel: every token of the batch against the keys of ITS sequence that lie in the same chunk of `chunk` positions
//     (chunks counted from position 0 of the sequence) and not after it; softmax with a per-head sink logit in the denominator; sigmoid
//     output gate.  Prompt portions and single decoded tokens are the same case: a token is (sequence, position), its keys are looked up
//     through the sequence's block-table row, and the rows a call appends are in the pool before the scores are formed.
// Scores, softmax and the weighted sum are fp32; q, k, v and the output are of the engine dtype.
#include "hybrid_ops.cuh"

namespace b200 {

constexpr int kPage = B200_KV_PAGE_SIZE;

template <typename T>
__global__ void __launch_bounds__(256)
attn_qk_norm_cache_kernel(const T *__restrict__ proj, int ld, T *__restrict__ q_out, T *__restrict__ k_pool, T *__restrict__ v_pool,
                          const float *__restrict__ q_norm, const float *__restrict__ k_norm, float eps, const int *__restrict__ tok_seq,
                          const int *__restrict__ tok_pos, const int *__restrict__ block_table, int mpps, int heads, int kv_heads, int dim) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int nq = heads * dim, nk = kv_heads * dim;
    const T *row = proj + (size_t)t * ld;
    float sq = 0.0f, sk = 0.0f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float v = Elem<T>::to_f(row[c]);
        sq = fmaf(v, v, sq);
    }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const float v = Elem<T>::to_f(row[nq + c]);
        sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float iq = q_norm ? rsqrtf(sq / (float)nq + eps) : 1.0f;
    const float ik = k_norm ? rsqrtf(sk / (float)nk + eps) : 1.0f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float v = Elem<T>::to_f(row[c]);
        q_out[(size_t)t * nq + c] = Elem<T>::from_f(q_norm ? v * iq * q_norm[c] : v);
    }
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)tok_seq[t] * mpps + pos / kPage];
    if (page < 0) return;  // no page held: nothing is written (the host refuses such a batch)
    const int off = pos % kPage;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const int g = c / dim, cc = c - g * dim;
        const float v = Elem<T>::to_f(row[nq + c]);
        const size_t at = (((size_t)page * kv_heads + g) * kPage + off) * dim + cc;
        k_pool[at] = Elem<T>::from_f(k_norm ? v * ik * k_norm[c] : v);
        v_pool[at] = row[nq + c];
    }
}

// One CTA per (token, query head).  Shared memory: q[dim] | scores[keys] | partial[groups][dim] | red[33].
template <typename T>
__global__ void __launch_bounds__(128)
chunked_attn_kernel(const T *__restrict__ q, const T *__restrict__ k_pool, const T *__restrict__ v_pool, const float *__restrict__ sink,
                    const T *__restrict__ gate_in, int gate_ld, T *__restrict__ out, const int *__restrict__ tok_seq,
                    const int *__restrict__ tok_pos, const int *__restrict__ block_table, int mpps, int heads, int kv_heads, int dim,
                    float scale, int chunk, int max_keys) {
    extern __shared__ float sm[];
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (heads / kv_heads);
    const int pos = tok_pos[t];
    const int first = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int nkeys = pos - first + 1;
    const int ngroups = (int)blockDim.x >= dim ? (int)blockDim.x / dim : 1;
    float *qs = sm;
    float *sc = qs + dim;
    float *part = sc + max_keys;
    float *red = part + (size_t)ngroups * dim;
    const int *bt = block_table + (size_t)tok_seq[t] * mpps;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) qs[c] = Elem<T>::to_f(q[((size_t)t * heads + h) * dim + c]);
    __syncthreads();

    // ---- scores: one key per thread
    const bool vec = (dim % Elem<T>::kVec) == 0;
    float mx = sink ? sink[h] : -INFINITY;
    for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
        const int p = first + j;
        const int page = bt[p / kPage];
        const T *kr = k_pool + (((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim;
        float acc = 0.0f;
        if (vec) {
            constexpr int V = Elem<T>::kVec;
            for (int c = 0; c < dim; c += V) {
                float f[V];
                unpack16<T>(ld_v4(kr + c), f);
#pragma unroll
                for (int i = 0; i < V; ++i) acc = fmaf(qs[c + i], f[i], acc);
            }
        } else {
            for (int c = 0; c < dim; ++c) acc = fmaf(qs[c], Elem<T>::to_f(kr[c]), acc);
        }
        acc *= scale;
        sc[j] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    sum = block_sum(sum, red);  // (its barriers also publish sc[])
    if (sink) sum += expf(sink[h] - mx);
    const float inv = 1.0f / sum;

    // ---- weighted sum of the values: column c by thread, keys dealt over `ngroups` thread groups
    if (ngroups > 1) {
        const int kg = threadIdx.x / dim, c = threadIdx.x - kg * dim;
        if (kg < ngroups) {
            float acc = 0.0f;
            for (int j = kg; j < nkeys; j += ngroups) {
                const int p = first + j;
                const int page = bt[p / kPage];
                acc = fmaf(sc[j], Elem<T>::to_f(v_pool[(((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim + c]), acc);
            }
            part[kg * dim + c] = acc;
        }
        __syncthreads();
        if ((int)threadIdx.x < dim) {
            float acc = 0.0f;
            for (int k2 = 0; k2 < ngroups; ++k2) acc += part[k2 * dim + threadIdx.x];
            part[threadIdx.x] = acc;
        }
        __syncthreads();
    } else {
        for (int c = threadIdx.x; c < dim; c += blockDim.x) {
            float acc = 0.0f;
            for (int j = 0; j < nkeys; ++j) {
                const int p = first + j;
                const int page = bt[p / kPage];
                acc = fmaf(sc[j], Elem<T>::to_f(v_pool[(((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim + c]), acc);
            }
            part[c] = acc;
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float o = part[c] * inv;
        if (gate_in) {
            const float z = Elem<T>::to_f(gate_in[(size_t)t * gate_ld + h * dim + c]);
            o *= 1.0f / (1.0f + expf(-z));
        }
        out[((size_t)t * heads + h) * dim + c] = Elem<T>::from_f(o);
    }
}

int launch_attn_qk_norm_cache(int dtype, const void *proj, int ld, void *q_out, void *k_pool, void *v_pool, const float *q_norm,
                              const float *k_norm, float eps, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps,
                              int tokens, int heads, int kv_heads, int dim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        attn_qk_norm_cache_kernel<T><<<tokens, 256, 0, st>>>((const T *)proj, ld, (T *)q_out, (T *)k_pool, (T *)v_pool, q_norm, k_norm, eps,
                                                              tok_seq, tok_pos, block_table, mpps, heads, kv_heads, dim);
    });
    return cuda_status("attn_qk_norm_cache launch");
}

int launch_chunked_attention(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                             int gate_ld, void *out, const int *tok_seq, const int *tok_pos, const int *block_table, int mpps, int tokens,
                             int heads, int kv_heads, int dim, float scale, int chunk, int max_keys, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const int threads = 128;
    const int ngroups = threads >= dim ? threads / dim : 1;
    const size_t smem = ((size_t)dim + max_keys + (size_t)ngroups * dim + 33) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("chunked_attention: %d keys x dim %d do not fit the shared-memory score buffer", max_keys, dim);
        return B200_ERR_UNSUPPORTED;
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(chunked_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        chunked_attn_kernel<T><<<dim3(tokens, heads), threads, smem, st>>>((const T *)q, (const T *)k_pool, (const T *)v_pool, sink,
                                                                            (const T *)gate_in, gate_ld, (T *)out, tok_seq, tok_pos,
                                                                            block_table, mpps, heads, kv_heads, dim, scale, chunk, max_keys);
    });
    return cuda_status("chunked_attention launch");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_attn_qk_norm_cache_paged(const void *proj, int ld, void *q_out, void *k_pool, void *v_pool, const float *q_norm,
                                  const float *k_norm, float eps, const int *tok_seq, const int *tok_pos, const int *block_table,
                                  int max_pages_per_seq, int tokens, int heads, int kv_heads, int dim, int dtype, b200_stream_t stream) {
    B200_REQUIRE(proj && q_out && k_pool && v_pool && tok_seq && tok_pos && block_table, "attn_qk_norm_cache: null pointer");
    B200_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && ld >= (heads + kv_heads) * dim, "attn_qk_norm_cache: bad shape");
    return launch_attn_qk_norm_cache(dtype, proj, ld, q_out, k_pool, v_pool, q_norm, k_norm, eps, tok_seq, tok_pos, block_table,
                                     max_pages_per_seq, tokens, heads, kv_heads, dim, as_stream(stream));
}

int b200_chunked_attention_paged(const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                                 int gate_ld, void *out, const int *tok_seq, const int *tok_pos, const int *block_table,
                                 int max_pages_per_seq, int tokens, int heads, int kv_heads, int dim, float scale, int chunk,
                                 int dtype, b200_stream_t stream) {
    B200_REQUIRE(q && k_pool && v_pool && out && tok_seq && tok_pos && block_table, "chunked_attention: null pointer");
    B200_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && chunk >= 0, "chunked_attention: bad shape");
    const int max_keys = chunk > 0 ? chunk : max_pages_per_seq * kPage;
    return launch_chunked_attention(dtype, q, k_pool, v_pool, sink, gate_in, gate_ld, out, tok_seq, tok_pos, block_table,
                                    max_pages_per_seq, tokens, heads, kv_heads, dim, scale, chunk, max_keys, as_stream(stream));
}
}
