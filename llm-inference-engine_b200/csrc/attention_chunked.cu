// attention_chunked.cu -- softmax attention without rotation over a paged key/value pool, for ragged mixed batches:
//   * attn_qk_norm_cache_kernel: RMS norm over the WHOLE q projection and the WHOLE k projection (all heads at once), q to a dense
//     buffer, normed k to the K pool, k as projected to the V pool (the values of this mixer are its un-normed keys);
//   * chunked_attn_kernel: every token of the batch against the keys of ITS sequence that lie in the same chunk of `chunk` positions
//     (chunks counted from position 0 of the sequence) and not after it; softmax with a per-head sink logit in the denominator; sigmoid
//     output gate.  Prompt portions and single decoded tokens are the same case: a token is (sequence, position), its keys are looked up
//     through the sequence's block-table row, and the rows a call appends are in the pool before the scores are formed.
// Scores, softmax and the weighted sum are fp32; q, k, v and the output are of the engine dtype.
#include "hybrid_ops.cuh"

#include <algorithm>

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
    constexpr int V = Elem<T>::kVec;
    // 16-byte pieces when rows, heads and the pools' rows all start on 16-byte boundaries
    const bool vec = nq % V == 0 && dim % V == 0 && ld % V == 0 &&
                     ((reinterpret_cast<size_t>(proj) | reinterpret_cast<size_t>(q_out) | reinterpret_cast<size_t>(k_pool) |
                       reinterpret_cast<size_t>(v_pool) | reinterpret_cast<size_t>(q_norm) | reinterpret_cast<size_t>(k_norm)) & 15) == 0;
    float sq = 0.0f, sk = 0.0f;
    if (vec) {
        for (int c = threadIdx.x * V; c < nq + nk; c += blockDim.x * V) {  // nq is a multiple of V: a piece is all q or all k
            float f[V];
            unpack16<T>(ld_v4(row + c), f);
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < V; ++e) ss = fmaf(f[e], f[e], ss);
            if (c < nq) sq += ss; else sk += ss;
        }
    } else {
        for (int c = threadIdx.x; c < nq; c += blockDim.x) {
            const float v = Elem<T>::to_f(row[c]);
            sq = fmaf(v, v, sq);
        }
        for (int c = threadIdx.x; c < nk; c += blockDim.x) {
            const float v = Elem<T>::to_f(row[nq + c]);
            sk = fmaf(v, v, sk);
        }
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float iq = q_norm ? rsqrtf(sq / (float)nq + eps) : 1.0f;
    const float ik = k_norm ? rsqrtf(sk / (float)nk + eps) : 1.0f;
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)tok_seq[t] * mpps + pos / kPage];
    const int off = pos % kPage;
    if (vec) {
        for (int c = threadIdx.x * V; c < nq + nk; c += blockDim.x * V) {
            const uint4 raw = ld_v4(row + c);
            float f[V];
            unpack16<T>(raw, f);
            const bool is_q = c < nq;
            const float *nw = is_q ? q_norm : k_norm;
            if (nw) {
                const float inv = is_q ? iq : ik;
                const int cn = is_q ? c : c - nq;
#pragma unroll
                for (int e = 0; e < V; ++e) f[e] = f[e] * inv * nw[cn + e];
            }
            if (is_q) {
                st_v4(q_out + (size_t)t * nq + c, nw ? pack16<T>(f) : raw);
            } else if (page >= 0) {  // no page held: nothing is written (the host refuses such a batch)
                const int ck = c - nq, g = ck / dim, cc = ck - g * dim;
                const size_t at = (((size_t)page * kv_heads + g) * kPage + off) * dim + cc;
                st_v4(k_pool + at, nw ? pack16<T>(f) : raw);
                st_v4(v_pool + at, raw);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float v = Elem<T>::to_f(row[c]);
        q_out[(size_t)t * nq + c] = Elem<T>::from_f(q_norm ? v * iq * q_norm[c] : v);
    }
    if (page < 0) return;  // no page held: nothing is written (the host refuses such a batch)
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const int g = c / dim, cc = c - g * dim;
        const float v = Elem<T>::to_f(row[nq + c]);
        const size_t at = (((size_t)page * kv_heads + g) * kPage + off) * dim + cc;
        k_pool[at] = Elem<T>::from_f(k_norm ? v * ik * k_norm[c] : v);
        v_pool[at] = row[nq + c];
    }
}

// One CTA per (token, query head).  Shared memory: q[dim] | scores[keys] | partial[key groups][dim] | red[33].
template <typename T>
__global__ void __launch_bounds__(512)
chunked_attn_kernel(const T *__restrict__ q, const T *__restrict__ k_pool, const T *__restrict__ v_pool, const float *__restrict__ sink,
                    const T *__restrict__ gate_in, int gate_ld, T *__restrict__ out, const int *__restrict__ tok_seq,
                    const int *__restrict__ tok_pos, const int *__restrict__ block_table, int mpps, int heads, int kv_heads, int dim,
                    float scale, int chunk, int max_keys, const int *__restrict__ tok_list) {
    extern __shared__ float sm[];
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    const int g = h / (heads / kv_heads);
    const int pos = tok_pos[t];
    const int first = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int nkeys = pos - first + 1;
    const int ngroups = (int)blockDim.x >= dim ? (int)blockDim.x / dim : 1;
    float *qs = sm;
    float *sc = qs + dim;
    float *part = sc + max_keys;
    float *red = part + max((size_t)ngroups * dim, (size_t)blockDim.x * 8);
    const int *bt = block_table + (size_t)tok_seq[t] * mpps;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) qs[c] = Elem<T>::to_f(q[((size_t)t * heads + h) * dim + c]);
    __syncthreads();

    // ---- scores: four adjacent lanes share a key row (each takes every fourth 16-byte piece, so a warp's load covers whole 64-byte
    // segments of eight rows and a short chunk still spreads over the block); other head sizes: one key per thread
    const bool vec = (dim % Elem<T>::kVec) == 0;
    float mx = sink ? sink[h] : -INFINITY;
    if (dim % (4 * Elem<T>::kVec) == 0 && blockDim.x % 32 == 0) {
        constexpr int V = Elem<T>::kVec;
        const int sub = threadIdx.x & 3, kslot = threadIdx.x >> 2, nslots = blockDim.x >> 2, pieces = dim / V;
#pragma unroll 2
        for (int j0 = 0; j0 < nkeys; j0 += nslots) {  // warp-uniform trip count: the shuffles below take every lane
            const int j = j0 + kslot;
            const int p = first + min(j, nkeys - 1);
            const int page = bt[p / kPage];
            const T *kr = k_pool + (((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim;
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
            for (int pc = sub; pc < pieces; pc += 4) {
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
            acc *= scale;
            if (j < nkeys) {
                if (sub == 0) sc[j] = acc;
                mx = fmaxf(mx, acc);
            }
        }
    } else {
        for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
            const int p = first + j;
            const int page = bt[p / kPage];
            const T *kr = k_pool + (((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim;
            float acc = 0.0f;
            if (vec) {
                constexpr int V = Elem<T>::kVec;
#pragma unroll 8
                for (int c = 0; c < dim; c += V) {  // unrolled: a thread's loads of one key row are in flight together
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

    // ---- weighted sum of the values
    constexpr int V = Elem<T>::kVec;
    const int tpr = dim / V;  // threads per value row when a thread takes one 16-byte piece
    if (vec && tpr <= (int)blockDim.x) {
        // a thread owns V consecutive columns; the block walks blockDim / tpr keys at a time with 16-byte loads, then the key groups'
        // partial sums meet in shared memory
        const int groups = (int)blockDim.x / tpr, kg = threadIdx.x / tpr, c0 = (threadIdx.x - kg * tpr) * V;
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.0f;
        if (kg < groups) {
#pragma unroll 8
            for (int j = kg; j < nkeys; j += groups) {
                const int p = first + j;
                const int page = bt[p / kPage];
                float f[V];
                unpack16<T>(ld_v4(v_pool + (((size_t)page * kv_heads + g) * kPage + (p % kPage)) * dim + c0), f);
                const float w = sc[j];
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(w, f[i], acc[i]);
            }
#pragma unroll
            for (int i = 0; i < V; ++i) part[kg * dim + c0 + i] = acc[i];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < dim; c += blockDim.x) {
            float a = 0.0f;
            for (int k2 = 0; k2 < groups; ++k2) a += part[k2 * dim + c];
            part[c] = a;  // column c's entries are read by this thread only
        }
        __syncthreads();
    } else if (ngroups > 1) {
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

// ---------------------------------------------------------------------------------------------------------------------------------
// Tensor-core prefill kernel (16-bit engines, dim 64 or 128): one CTA = 64 consecutive tokens of ONE sequence x one query head, four
// warps of 16 rows each.  A key tile is one page (64 positions): K and V arrive by cp.async into a two-stage ring, S = Q K^T and
// O += P V run on mma.sync.m16n8k16 with fp32 accumulators, the softmax is the online form in fp32.  The sink enters as the INITIAL
// running state (max = sink, sum = 1, nothing accumulated): exactly a key with that logit and a zero value, and it keeps the running
// max finite for rows whose first tiles are masked out entirely.  The mask is evaluated per element, so a tile of queries may straddle a
// chunk edge; the tiles walked are those from the chunk start of the tile's first query to its last query.
// tiles: int4 per tile {sequence, first packed row, rows (1..64), position of the first row}.
constexpr int kTileQ = 64;

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
template <typename T> __device__ __forceinline__ void mma_16816(float *c, const unsigned *a, unsigned b0, unsigned b1);
template <> __device__ __forceinline__ void mma_16816<__nv_bfloat16>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16816<__half>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ unsigned pack2(float lo, float hi);
template <> __device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}
template <> __device__ __forceinline__ unsigned pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}

// element (row, col) of a [rows][D] 16-bit tile whose 16-byte pieces are XOR-swizzled by the row: conflict-free ldmatrix
template <int D> __device__ __forceinline__ int swz(int row, int col) { return row * D + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)); }

template <typename T, int D>
__global__ void __launch_bounds__(128)
chunked_attn_mma_kernel(const T *__restrict__ q, const T *__restrict__ k_pool, const T *__restrict__ v_pool, const float *__restrict__ sink,
                        const T *__restrict__ gate_in, int gate_ld, T *__restrict__ out, const int4 *__restrict__ tiles,
                        const int *__restrict__ block_table, int mpps, int heads, int kv_heads, float scale, int chunk) {
    extern __shared__ __align__(16) unsigned char smraw[];
    T *qs = reinterpret_cast<T *>(smraw);     // [64][D]
    T *ks = qs + kTileQ * D;                  // [2][64][D]
    T *vs = ks + 2 * kPage * D;               // [2][64][D]
    const int4 tile = tiles[blockIdx.x];
    const int h = blockIdx.y, g = h / (heads / kv_heads);
    const int row0 = tile.y, nrows = tile.z, pos0 = tile.w;
    const int *bt = block_table + (size_t)tile.x * mpps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    constexpr int kPieces = D / 8;            // 16-byte pieces per row

    const int last = pos0 + nrows - 1;
    const int first = chunk > 0 ? (pos0 / chunk) * chunk : 0;
    const int tile_lo = first / kPage, tile_hi = last / kPage;

    auto load_kv = [&](int kt, int stage) {
        const int page = bt[kt];
        const T *kg = k_pool + ((size_t)page * kv_heads + g) * kPage * D;
        const T *vg = v_pool + ((size_t)page * kv_heads + g) * kPage * D;
        for (int i = threadIdx.x; i < kPage * kPieces; i += 128) {
            const int r = i / kPieces, c = (i % kPieces) * 8;
            cp_async16(ks + stage * kPage * D + swz<D>(r, c), kg + r * D + c);
            // rows past the tile's last query have not been written (or belong to a page's previous owner): their probabilities are
            // zero, but 0 x NaN is NaN on the tensor core, so the values are zeroed rather than fetched
            if (kt * kPage + r <= last) cp_async16(vs + stage * kPage * D + swz<D>(r, c), vg + r * D + c);
            else *reinterpret_cast<uint4 *>(vs + stage * kPage * D + swz<D>(r, c)) = make_uint4(0, 0, 0, 0);
        }
    };
    load_kv(tile_lo, 0);
    cp_async_commit();
    for (int i = threadIdx.x; i < kTileQ * kPieces; i += 128) {
        const int r = i / kPieces, c = (i % kPieces) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) v = ld_v4(q + ((size_t)(row0 + r) * heads + h) * D + c);
        *reinterpret_cast<uint4 *>(qs + swz<D>(r, c)) = v;
    }
    __syncthreads();
    unsigned qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldsm_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + swz<D>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 16 + (lane >> 4) * 8));

    constexpr float kLog2e = 1.4426950408889634f;
    const float sl2 = scale * kLog2e;
    // rows gid and gid + 8 of this warp's 16
    const int p_a = pos0 + warp * 16 + gid, p_b = p_a + 8;
    const int c_a = chunk > 0 ? p_a / chunk : 0, c_b = chunk > 0 ? p_b / chunk : 0;
    float m_a, m_b, l_a, l_b;
    if (sink) m_a = m_b = sink[h] * kLog2e, l_a = l_b = tig == 0 ? 1.0f : 0.0f;  // the sum is kept per lane and joined at the end
    else m_a = m_b = -1e30f, l_a = l_b = 0.0f;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    for (int kt = tile_lo; kt <= tile_hi; ++kt) {
        const int stage = (kt - tile_lo) & 1;
        if (kt < tile_hi) load_kv(kt + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const T *kst = ks + stage * kPage * D, *vst = vs + stage * kPage * D;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {  // two key blocks of 8 per ldmatrix
                unsigned b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, kst + swz<D>(jp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8));
                mma_16816<T>(s[2 * jp], qf[kk], b0, b1);
                mma_16816<T>(s[2 * jp + 1], qf[kk], b2, b3);
            }
        }
        // scale, mask, running max
        float mx_a = m_a, mx_b = m_b;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kt * kPage + j * 8 + tig * 2 + e;
                const int kc = chunk > 0 ? key / chunk : 0;
                s[j][e] = (key <= p_a && kc == c_a) ? s[j][e] * sl2 : -INFINITY;
                s[j][2 + e] = (key <= p_b && kc == c_b) ? s[j][2 + e] * sl2 : -INFINITY;
                mx_a = fmaxf(mx_a, s[j][e]);
                mx_b = fmaxf(mx_b, s[j][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float f_a = exp2f(m_a - mx_a), f_b = exp2f(m_b - mx_b);
        m_a = mx_a, m_b = mx_b;
        float sum_a = 0.0f, sum_b = 0.0f;
        unsigned pf[4][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float e0 = exp2f(s[j][0] - m_a), e1 = exp2f(s[j][1] - m_a), e2 = exp2f(s[j][2] - m_b), e3 = exp2f(s[j][3] - m_b);
            sum_a += e0 + e1, sum_b += e2 + e3;
            pf[j >> 1][(j & 1) * 2] = pack2<T>(e0, e1);
            pf[j >> 1][(j & 1) * 2 + 1] = pack2<T>(e2, e3);
        }
        l_a = l_a * f_a + sum_a, l_b = l_b * f_b + sum_b;  // per-lane partial sums; joined across the row's four lanes at the end
#pragma unroll
        for (int j = 0; j < D / 8; ++j) o[j][0] *= f_a, o[j][1] *= f_a, o[j][2] *= f_b, o[j][3] *= f_b;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
            for (int jp = 0; jp < D / 16; ++jp) {
                unsigned b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, vst + swz<D>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 16 + (lane >> 4) * 8));
                mma_16816<T>(o[2 * jp], pf[kk], b0, b1);
                mma_16816<T>(o[2 * jp + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();  // everybody is done with this stage before the next iteration's prefetch overwrites it
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float i_a = 1.0f / l_a, i_b = 1.0f / l_b;
    const int r_a = warp * 16 + gid, r_b = r_a + 8;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int c = j * 8 + tig * 2;
        if (r_a < nrows) {
            float x0 = o[j][0] * i_a, x1 = o[j][1] * i_a;
            if (gate_in) {
                const T *gp = gate_in + (size_t)(row0 + r_a) * gate_ld + h * D + c;
                x0 *= 1.0f / (1.0f + expf(-Elem<T>::to_f(gp[0]))), x1 *= 1.0f / (1.0f + expf(-Elem<T>::to_f(gp[1])));
            }
            *reinterpret_cast<unsigned *>(out + ((size_t)(row0 + r_a) * heads + h) * D + c) = pack2<T>(x0, x1);
        }
        if (r_b < nrows) {
            float x2 = o[j][2] * i_b, x3 = o[j][3] * i_b;
            if (gate_in) {
                const T *gp = gate_in + (size_t)(row0 + r_b) * gate_ld + h * D + c;
                x2 *= 1.0f / (1.0f + expf(-Elem<T>::to_f(gp[0]))), x3 *= 1.0f / (1.0f + expf(-Elem<T>::to_f(gp[1])));
            }
            *reinterpret_cast<unsigned *>(out + ((size_t)(row0 + r_b) * heads + h) * D + c) = pack2<T>(x2, x3);
        }
    }
}

template <typename T, int D>
static int launch_mma_t(const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in, int gate_ld, void *out,
                        const int *tiles, int n_tiles, const int *block_table, int mpps, int heads, int kv_heads, float scale, int chunk,
                        cudaStream_t st) {
    const size_t smem = (size_t)(kTileQ + 4 * kPage) * D * sizeof(T);
    cudaFuncSetAttribute(chunked_attn_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunked_attn_mma_kernel<T, D><<<dim3(n_tiles, heads), 128, smem, st>>>((const T *)q, (const T *)k_pool, (const T *)v_pool, sink, (const T *)gate_in,
                                                                            gate_ld, (T *)out, (const int4 *)tiles, block_table, mpps, heads, kv_heads,
                                                                            scale, chunk);
    return cuda_status("chunked_attention (tensor core) launch");
}

bool chunked_attention_tiles_supported(int dtype, int dim, int gate_ld) {
    return dtype != B200_F32 && (dim == 64 || dim == 128) && gate_ld % 2 == 0;
}

int launch_chunked_attention_tiles(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                                   int gate_ld, void *out, const int *tiles, int n_tiles, const int *block_table, int mpps, int heads,
                                   int kv_heads, int dim, float scale, int chunk, cudaStream_t st) {
    if (n_tiles == 0) return B200_OK;
    if (!chunked_attention_tiles_supported(dtype, dim, gate_ld)) {
        set_error("chunked_attention tiles: 16-bit dtypes and dim 64 / 128 only");
        return B200_ERR_UNSUPPORTED;
    }
#define B200_ATTN_TILES(TT, DD) \
    return launch_mma_t<TT, DD>(q, k_pool, v_pool, sink, gate_in, gate_ld, out, tiles, n_tiles, block_table, mpps, heads, kv_heads, scale, chunk, st)
    if (dtype == B200_BF16) {
        if (dim == 64) B200_ATTN_TILES(__nv_bfloat16, 64);
        B200_ATTN_TILES(__nv_bfloat16, 128);
    }
    if (dim == 64) B200_ATTN_TILES(__half, 64);
    B200_ATTN_TILES(__half, 128);
#undef B200_ATTN_TILES
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
                             int heads, int kv_heads, int dim, float scale, int chunk, int max_keys, cudaStream_t st, const int *tok_list) {
    if (tokens == 0) return B200_OK;
    const int threads = max_keys >= 512 ? 512 : (max_keys >= 256 ? 256 : 128);  // long chunks: more keys in flight per CTA
    const int ngroups = threads >= dim ? threads / dim : 1;
    const size_t part = std::max((size_t)ngroups * dim, (size_t)threads * 8);  // key-group partial sums (scalar / 16-byte path)
    const size_t smem = ((size_t)dim + max_keys + part + 33) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("chunked_attention: %d keys x dim %d do not fit the shared-memory score buffer", max_keys, dim);
        return B200_ERR_UNSUPPORTED;
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(chunked_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        chunked_attn_kernel<T><<<dim3(tokens, heads), threads, smem, st>>>((const T *)q, (const T *)k_pool, (const T *)v_pool, sink,
                                                                            (const T *)gate_in, gate_ld, (T *)out, tok_seq, tok_pos,
                                                                            block_table, mpps, heads, kv_heads, dim, scale, chunk, max_keys, tok_list);
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
                                    max_pages_per_seq, tokens, heads, kv_heads, dim, scale, chunk, max_keys, as_stream(stream), nullptr);
}

int b200_chunked_attention_prefill_paged(const void *q, const void *k_pool, const void *v_pool, const float *sink, const void *gate_in,
                                         int gate_ld, void *out, const int *tiles, int n_tiles, const int *block_table,
                                         int max_pages_per_seq, int heads, int kv_heads, int dim, float scale, int chunk, int dtype,
                                         b200_stream_t stream) {
    B200_REQUIRE(q && k_pool && v_pool && out && tiles && block_table, "chunked_attention_prefill: null pointer");
    B200_REQUIRE(n_tiles >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && chunk >= 0, "chunked_attention_prefill: bad shape");
    B200_REQUIRE(((uintptr_t)tiles & 15) == 0, "chunked_attention_prefill: the tile list must be 16-byte aligned");
    return launch_chunked_attention_tiles(dtype, q, k_pool, v_pool, sink, gate_in, gate_ld, out, tiles, n_tiles, block_table, max_pages_per_seq,
                                          heads, kv_heads, dim, scale, chunk, as_stream(stream));
}
}
