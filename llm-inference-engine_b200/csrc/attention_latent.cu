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
    constexpr int V = Elem<T>::kVec;
    if (dim % V == 0 && rot_dim % V == 0 && ld % V == 0 && q_col % V == 0 &&
        ((reinterpret_cast<size_t>(proj) | reinterpret_cast<size_t>(qn)) & 15) == 0) {  // the un-rotated part moves in 16-byte pieces
        const int pieces = dim / V;
        for (int idx = threadIdx.x; idx < heads * pieces; idx += blockDim.x) {
            const int h = idx / pieces, c = (idx - h * pieces) * V;
            st_v4(qn + ((size_t)h * t_pad + t) * dim + c, ld_v4(row + q_col + (size_t)h * per + c));
        }
        for (int idx = threadIdx.x; idx < heads * rot_dim; idx += blockDim.x) {
            const int h = idx / rot_dim, r = idx - h * rot_dim;
            qr[((size_t)t * heads + h) * rot_dim + r] = Elem<T>::from_f(rotated(row + q_col + (size_t)h * per + dim, r));
        }
    } else {
        for (int idx = threadIdx.x; idx < heads * per; idx += blockDim.x) {
            const int h = idx / per, c = idx - h * per;
            const T *qh = row + q_col + (size_t)h * per;
            if (c < dim) qn[((size_t)h * t_pad + t) * dim + c] = qh[c];
            else qr[((size_t)t * heads + h) * rot_dim + (c - dim)] = Elem<T>::from_f(rotated(qh + dim, c - dim));
        }
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

// ---------------------------------------------------------------------------------------------------------------------------------
// Tensor-core kernel (16-bit engines; kv_rank and rot_dim multiples of 16): one CTA = a tile of <= 64 query rows that share their keys,
// four warps of 16 rows each.  Two kinds of tile:
//   by_head == 0: 64 consecutive tokens of ONE sequence x one head (blockIdx.y)          -- prompt portions;
//   by_head == 1: ONE token x 64 consecutive heads (blockIdx.y * 64 ...)                  -- decoded tokens of many-headed layers: the
//                 heads share every key row, so the window is read once per 64 heads instead of once per head.
// A key tile is one page (64 positions) of rows [c | kr]: it arrives by cp.async into a two-stage ring, S = Q K^T over all kv_rank +
// rot_dim columns and O += P V over value columns [v0, v0 + 16 NV) OF THE SAME TILE run on mma.sync.m16n8k16 with fp32 accumulators, the
// softmax is the online form in fp32.  A CTA accumulates the whole rank up to 256 value columns; above that blockIdx.z selects a block of
// 128 value columns (the scores are formed again per block).  The sink enters as the INITIAL running state (max = sink, sum = 1, nothing accumulated): a key with that logit and a
// zero value.  The mask is evaluated per element: a tile of queries may straddle a window edge; the key tiles walked run from the
// window start of the tile's first query to its last query.  Rows of a key tile past the tile's last query are zeroed, not fetched:
// they may belong to a page's previous owner, and 0 x NaN is NaN on the tensor core.
// One-token tiles that would leave most of the device idle share out their key tiles over `splits` CTAs (blockIdx.z % splits), which write
// un-normalised sums and their running state to `part`; latent_combine_kernel joins them.  The sink belongs to share 0.
// tiles: int4 per tile {sequence, first packed row, rows (1..64; by_head: unused), position of the first row}.
namespace {
__device__ __forceinline__ void lat_cp_async16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void lat_ldsm_x4(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void lat_ldsm_x4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
template <typename T> __device__ __forceinline__ void lat_mma(float *c, const unsigned *a, unsigned b0, unsigned b1);
template <> __device__ __forceinline__ void lat_mma<__nv_bfloat16>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void lat_mma<__half>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ unsigned lat_pack2(float lo, float hi);
template <> __device__ __forceinline__ unsigned lat_pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}
template <> __device__ __forceinline__ unsigned lat_pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}
// element (row, col) of a [rows][ld] 16-bit tile (ld a multiple of 64) whose 16-byte pieces are XOR-swizzled by the row within groups of
// eight pieces: conflict-free ldmatrix
__device__ __forceinline__ int lat_swz(int row, int col, int ld) { return row * ld + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)); }
constexpr int kLatTileQ = 64;
constexpr int kLatentFillCtas = 148;
}  // namespace

template <typename T, int NV>
__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(const T *__restrict__ ql, const T *__restrict__ qr, const T *__restrict__ pool, const float *__restrict__ sink,
                       T *__restrict__ ol, const int4 *__restrict__ tiles, const int *__restrict__ block_table, int mpps, int t_pad, int heads,
                       int kv_rank, int rot_dim, int ld, float scale, int window, int by_head, int splits, float *__restrict__ part) {
    extern __shared__ __align__(16) unsigned char smraw[];
    T *qs = reinterpret_cast<T *>(smraw);  // [64][ld]
    T *ks = qs + kLatTileQ * ld;           // [2][64][ld]
    const int4 tile = tiles[blockIdx.x];
    const int dk = kv_rank + rot_dim, pieces = dk / 8;
    const int row0 = tile.y, pos0 = tile.w;
    const int h0 = by_head ? blockIdx.y * kLatTileQ : blockIdx.y;
    const int nrows = by_head ? min(kLatTileQ, heads - h0) : tile.z;
    const int sp = blockIdx.z % splits;  // which share of the key tiles this CTA walks (splits > 1: partial results go to `part`)
    const int v0 = (blockIdx.z / splits) * (16 * NV);
    const int *bt = block_table + (size_t)tile.x * mpps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int last = by_head ? pos0 : pos0 + nrows - 1;
    const int first = window > 0 ? max(0, pos0 - window + 1) : 0;
    int tile_lo = first / kPageL, tile_hi = last / kPageL;
    if (splits > 1) {
        const int per = (tile_hi - tile_lo + splits) / splits;
        tile_lo += sp * per;
        tile_hi = min(tile_hi, tile_lo + per - 1);  // may leave no tile: this CTA then reports an empty share
    }

    auto load_kv = [&](int kt, int stage) {
        const T *src = pool + (size_t)bt[kt] * kPageL * dk;
        T *dst = ks + stage * kPageL * ld;
        for (int i = threadIdx.x; i < kPageL * pieces; i += 128) {
            const int r = i / pieces, c = (i - r * pieces) * 8;
            if (kt * kPageL + r <= last) lat_cp_async16(dst + lat_swz(r, c, ld), src + (size_t)r * dk + c);
            else *reinterpret_cast<uint4 *>(dst + lat_swz(r, c, ld)) = make_uint4(0, 0, 0, 0);
        }
    };
    if (tile_lo <= tile_hi) load_kv(tile_lo, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = threadIdx.x; i < kLatTileQ * pieces; i += 128) {
        const int r = i / pieces, c = (i - r * pieces) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) {
            const int t = by_head ? row0 : row0 + r, h = by_head ? h0 + r : h0;
            v = c < kv_rank ? ld_v4(ql + ((size_t)h * t_pad + t) * kv_rank + c) : ld_v4(qr + ((size_t)t * heads + h) * rot_dim + (c - kv_rank));
        }
        *reinterpret_cast<uint4 *>(qs + lat_swz(r, c, ld)) = v;
    }

    constexpr float kLog2e = 1.4426950408889634f;
    const float sl2 = scale * kLog2e;
    // rows gid and gid + 8 of this warp's 16
    const int r_a = warp * 16 + gid, r_b = r_a + 8;
    const int p_a = by_head ? pos0 : pos0 + r_a, p_b = by_head ? pos0 : pos0 + r_b;
    const int lo_a = window > 0 ? p_a - window : -1, lo_b = window > 0 ? p_b - window : -1;  // visible keys: lo < key <= p
    float m_a, m_b, l_a, l_b;
    if (sink && sp == 0) {
        m_a = sink[by_head ? min(h0 + r_a, heads - 1) : h0] * kLog2e, m_b = sink[by_head ? min(h0 + r_b, heads - 1) : h0] * kLog2e;
        l_a = l_b = tig == 0 ? 1.0f : 0.0f;  // the sum is kept per lane and joined at the end
    } else {
        m_a = m_b = -1e30f, l_a = l_b = 0.0f;
    }
    float o[2 * NV][4];
#pragma unroll
    for (int j = 0; j < 2 * NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    for (int kt = tile_lo; kt <= tile_hi; ++kt) {
        const int stage = (kt - tile_lo) & 1;
        if (kt < tile_hi) load_kv(kt + 1, stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const T *kst = ks + stage * kPageL * ld;
        if (warp * 16 >= nrows) {  // a warp without live rows only keeps the ring's barriers
            __syncthreads();
            continue;
        }
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll 2
        for (int kk = 0; kk < dk / 16; ++kk) {
            unsigned qf[4];
            lat_ldsm_x4(qf[0], qf[1], qf[2], qf[3], qs + lat_swz(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 16 + (lane >> 4) * 8, ld));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {  // two key blocks of 8 per ldmatrix
                unsigned b0, b1, b2, b3;
                lat_ldsm_x4(b0, b1, b2, b3, kst + lat_swz(jp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8, ld));
                lat_mma<T>(s[2 * jp], qf, b0, b1);
                lat_mma<T>(s[2 * jp + 1], qf, b2, b3);
            }
        }
        // scale, mask, running max
        float mx_a = m_a, mx_b = m_b;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kt * kPageL + j * 8 + tig * 2 + e;
                s[j][e] = (key <= p_a && key > lo_a) ? s[j][e] * sl2 : -INFINITY;
                s[j][2 + e] = (key <= p_b && key > lo_b) ? s[j][2 + e] * sl2 : -INFINITY;
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
            pf[j >> 1][(j & 1) * 2] = lat_pack2<T>(e0, e1);
            pf[j >> 1][(j & 1) * 2 + 1] = lat_pack2<T>(e2, e3);
        }
        l_a = l_a * f_a + sum_a, l_b = l_b * f_b + sum_b;  // per-lane partial sums; joined across the row's four lanes at the end
#pragma unroll
        for (int j = 0; j < 2 * NV; ++j) o[j][0] *= f_a, o[j][1] *= f_a, o[j][2] *= f_b, o[j][3] *= f_b;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step; the values are columns [v0, v0 + 16 NV) of the key tile itself
#pragma unroll
            for (int jp = 0; jp < NV; ++jp) {
                unsigned b0, b1, b2, b3;
                lat_ldsm_x4_trans(b0, b1, b2, b3, kst + lat_swz(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, v0 + jp * 16 + (lane >> 4) * 8, ld));
                lat_mma<T>(o[2 * jp], pf[kk], b0, b1);
                lat_mma<T>(o[2 * jp + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();  // everybody is done with this stage before the next iteration's prefetch overwrites it
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (part) {
        // a share of the keys: the un-normalised sums and the running state (max in log2 units, sum), fp32, per (tile, share, row):
        // [kv_rank sums | max | sum]; latent_combine_kernel joins the shares
        const size_t stride = (size_t)kv_rank + 2;
        float *pa = part + (((size_t)blockIdx.x * splits + sp) * heads + (by_head ? h0 + r_a : h0)) * stride;
        float *pb = part + (((size_t)blockIdx.x * splits + sp) * heads + (by_head ? h0 + r_b : h0)) * stride;
#pragma unroll
        for (int j = 0; j < 2 * NV; ++j) {
            const int c = v0 + j * 8 + tig * 2;
            if (r_a < nrows) pa[c] = o[j][0], pa[c + 1] = o[j][1];
            if (r_b < nrows) pb[c] = o[j][2], pb[c + 1] = o[j][3];
        }
        if (v0 == 0 && tig == 0) {
            if (r_a < nrows) pa[kv_rank] = m_a, pa[kv_rank + 1] = l_a;
            if (r_b < nrows) pb[kv_rank] = m_b, pb[kv_rank + 1] = l_b;
        }
        return;
    }
    const float i_a = 1.0f / l_a, i_b = 1.0f / l_b;
    T *out_a = ol + (by_head ? ((size_t)(h0 + r_a) * t_pad + row0) : ((size_t)h0 * t_pad + row0 + r_a)) * kv_rank + v0;
    T *out_b = ol + (by_head ? ((size_t)(h0 + r_b) * t_pad + row0) : ((size_t)h0 * t_pad + row0 + r_b)) * kv_rank + v0;
#pragma unroll
    for (int j = 0; j < 2 * NV; ++j) {
        const int c = j * 8 + tig * 2;
        if (r_a < nrows) *reinterpret_cast<unsigned *>(out_a + c) = lat_pack2<T>(o[j][0] * i_a, o[j][1] * i_a);
        if (r_b < nrows) *reinterpret_cast<unsigned *>(out_b + c) = lat_pack2<T>(o[j][2] * i_b, o[j][3] * i_b);
    }
}

// joins the shares of one-token tiles: grid (tiles, heads)
template <typename T>
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float *__restrict__ part, const int4 *__restrict__ tiles, T *__restrict__ ol, int t_pad, int heads, int kv_rank, int splits) {
    const int h = blockIdx.y, t = tiles[blockIdx.x].y;
    const size_t stride = (size_t)kv_rank + 2;
    const float *p0 = part + ((size_t)blockIdx.x * splits * heads + h) * stride;
    float w[8], mx = -INFINITY, den = 0.0f;  // splits <= 8
#pragma unroll
    for (int s = 0; s < 8; ++s) w[s] = s < splits ? p0[(size_t)s * heads * stride + kv_rank] : -INFINITY;
#pragma unroll
    for (int s = 0; s < 8; ++s) mx = fmaxf(mx, w[s]);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        w[s] = s < splits ? exp2f(w[s] - mx) : 0.0f;
        if (s < splits) den = fmaf(p0[(size_t)s * heads * stride + kv_rank + 1], w[s], den);
    }
    const float inv = 1.0f / den;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        float a = 0.0f;
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (s < splits) a = fmaf(p0[(size_t)s * heads * stride + c], w[s], a);
        ol[((size_t)h * t_pad + t) * kv_rank + c] = Elem<T>::from_f(a * inv);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
latent_gate_kernel(const T *__restrict__ ov, const T *__restrict__ gate_in, int gate_ld, T *__restrict__ out, int t_pad, int heads, int vdim) {
    const int t = blockIdx.x;
    constexpr int V = Elem<T>::kVec;
    if (vdim % V == 0 && gate_ld % V == 0 &&
        ((reinterpret_cast<size_t>(ov) | reinterpret_cast<size_t>(gate_in) | reinterpret_cast<size_t>(out)) & 15) == 0) {  // 16-byte pieces
        const int pieces = vdim / V;
        for (int idx = threadIdx.x; idx < heads * pieces; idx += blockDim.x) {
            const int h = idx / pieces, c = (idx - h * pieces) * V;
            float o[V], z[V];
            unpack16<T>(ld_v4(ov + ((size_t)h * t_pad + t) * vdim + c), o);
            unpack16<T>(ld_v4(gate_in + (size_t)t * gate_ld + h * vdim + c), z);
#pragma unroll
            for (int e = 0; e < V; ++e) o[e] = o[e] / (1.0f + expf(-z[e]));
            st_v4(out + ((size_t)t * heads + h) * vdim + c, pack16<T>(o));
        }
        return;
    }
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

// value blocks of 16 columns one CTA accumulates for this rank: the whole rank up to 256 columns (fp32 accumulators in registers), blocks of
// 128 (eight each, blockIdx.z of them) for larger ranks that are multiples of 128; 0: no tensor-core form
static int latent_value_blocks(int kv_rank) {
    if (kv_rank % 16 != 0) return 0;
    if (kv_rank <= 128 || (kv_rank <= 256 && kv_rank % 32 == 0)) return kv_rank / 16;
    return kv_rank % 128 == 0 ? 8 : 0;
}

bool latent_attention_tiles_supported(int dtype, int kv_rank, int rot_dim) {
    const int ld = (kv_rank + rot_dim + 63) / 64 * 64;
    return dtype != B200_F32 && rot_dim % 16 == 0 && latent_value_blocks(kv_rank) > 0 && (size_t)3 * kLatTileQ * ld * 2 <= 227 * 1024;
}

template <typename T, int NV>
static int launch_latent_mma_t(const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tiles, dim3 grid,
                               const int *block_table, int mpps, int t_pad, int heads, int kv_rank, int rot_dim, float scale, int window, int by_head,
                               int splits, float *part, cudaStream_t st) {
    const int ld = (kv_rank + rot_dim + 63) / 64 * 64;
    const size_t smem = (size_t)3 * kLatTileQ * ld * sizeof(T);
    cudaFuncSetAttribute(latent_attn_mma_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    latent_attn_mma_kernel<T, NV><<<grid, 128, smem, st>>>((const T *)ql, (const T *)qr, (const T *)pool, sink, (T *)ol, (const int4 *)tiles,
                                                           block_table, mpps, t_pad, heads, kv_rank, rot_dim, ld, scale, window, by_head, splits,
                                                           splits > 1 ? part : nullptr);
    if (splits > 1)
        latent_combine_kernel<T><<<dim3(grid.x, heads), 128, 0, st>>>(part, (const int4 *)tiles, (T *)ol, t_pad, heads, kv_rank, splits);
    return cuda_status("latent_attention (tensor core) launch");
}

int launch_latent_attention_tiles(int dtype, const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tiles,
                                  int n_tiles, const int *block_table, int mpps, int t_pad, int heads, int kv_rank, int rot_dim, float scale,
                                  int window, int by_head, float *part, int part_tiles, cudaStream_t st) {
    if (n_tiles == 0) return B200_OK;
    if (!latent_attention_tiles_supported(dtype, kv_rank, rot_dim)) {
        set_error("latent_attention tiles: 16-bit dtypes, kv_rank and rot_dim multiples of 16, kv_rank <= 128, a multiple of 32 up to 256, or a multiple of 128");
        return B200_ERR_UNSUPPORTED;
    }
    const int nv = latent_value_blocks(kv_rank);
    dim3 grid(n_tiles, by_head ? (heads + kLatTileQ - 1) / kLatTileQ : heads, kv_rank / (16 * nv));
    // one-token tiles that do not fill the device: the key tiles of every token are shared out over up to 8 CTAs, whose partial results
    // (part: fp32 [part_tiles, heads, kv_rank + 2]) a second kernel joins
    int splits = 1;
    if (by_head && part) {
        const int ctas = (int)(grid.x * grid.y * grid.z);
        if (ctas < kLatentFillCtas) splits = std::min(8, std::min(kLatentFillCtas / ctas, part_tiles / n_tiles));
        if (splits < 1) splits = 1;
    }
    grid.z *= splits;
#define B200_LAT_CASE(TT, N) \
    case N: return launch_latent_mma_t<TT, N>(ql, qr, pool, sink, ol, tiles, grid, block_table, mpps, t_pad, heads, kv_rank, rot_dim, scale, window, by_head, splits, part, st);
#define B200_LAT_TILES(TT)                                                                                                              \
    switch (nv) {                                                                                                                       \
        B200_LAT_CASE(TT, 1) B200_LAT_CASE(TT, 2) B200_LAT_CASE(TT, 3) B200_LAT_CASE(TT, 4) B200_LAT_CASE(TT, 5) B200_LAT_CASE(TT, 6)    \
        B200_LAT_CASE(TT, 7) B200_LAT_CASE(TT, 8) B200_LAT_CASE(TT, 10) B200_LAT_CASE(TT, 12) B200_LAT_CASE(TT, 14) B200_LAT_CASE(TT, 16) \
        default: break;                                                                                                                 \
    }
    if (dtype == B200_BF16) {
        B200_LAT_TILES(__nv_bfloat16)
    }
    B200_LAT_TILES(__half)
#undef B200_LAT_TILES
#undef B200_LAT_CASE
    set_error("latent_attention tiles: no kernel for rank %d", kv_rank);
    return B200_ERR_UNSUPPORTED;
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

using namespace b200;

extern "C" {

int b200_latent_prep_paged(const void *proj, int ld, int q_col, int kv_col, void *qn, void *qr, void *pool, const float *kv_norm, float eps,
                           const int *tok_seq, const int *tok_pos, const int *block_table, int max_pages_per_seq, int tokens, int t_pad,
                           int heads, int dim, int rot_dim, int kv_rank, int rot_dims, float rot_base, int dtype, b200_stream_t stream) {
    B200_REQUIRE(proj && qn && (qr || rot_dim == 0) && tok_seq && tok_pos && block_table, "latent_prep: null pointer");
    B200_REQUIRE(kv_col < 0 || (pool && kv_norm), "latent_prep: a layer that appends rows needs the pool and the row norm weight");
    B200_REQUIRE(tokens >= 0 && t_pad >= tokens && heads > 0 && dim > 0 && rot_dim >= 0 && kv_rank > 0 && q_col >= 0 &&
                     ld >= q_col + heads * (dim + rot_dim) && (kv_col < 0 || ld >= kv_col + kv_rank + rot_dim),
                 "latent_prep: bad shape");
    B200_REQUIRE(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 && (rot_dims == 0 || rot_base > 0.0f), "latent_prep: bad rotation");
    return launch_latent_prep(dtype, proj, ld, q_col, kv_col, qn, qr, pool, kv_norm, eps, tok_seq, tok_pos, block_table, max_pages_per_seq, tokens,
                              t_pad, heads, dim, rot_dim, kv_rank, rot_dims, rot_base, as_stream(stream));
}

int b200_latent_attention_paged(const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tok_seq,
                                const int *tok_pos, const int *block_table, int max_pages_per_seq, int tokens, int t_pad, int heads,
                                int kv_rank, int rot_dim, float scale, int window, int dtype, b200_stream_t stream) {
    B200_REQUIRE(ql && (qr || rot_dim == 0) && pool && ol && tok_seq && tok_pos && block_table, "latent_attention: null pointer");
    B200_REQUIRE(tokens >= 0 && t_pad >= tokens && heads > 0 && kv_rank > 0 && rot_dim >= 0 && window >= 0 && max_pages_per_seq > 0,
                 "latent_attention: bad shape");
    const int all = max_pages_per_seq * B200_KV_PAGE_SIZE;
    return launch_latent_attention(dtype, ql, qr, pool, sink, ol, tok_seq, tok_pos, block_table, max_pages_per_seq, tokens, t_pad, heads, kv_rank,
                                   rot_dim, scale, window, window > 0 ? std::min(window, all) : all, as_stream(stream), nullptr);
}

int b200_latent_attention_tiles_paged(const void *ql, const void *qr, const void *pool, const float *sink, void *ol, const int *tiles,
                                      int n_tiles, const int *block_table, int max_pages_per_seq, int t_pad, int heads, int kv_rank,
                                      int rot_dim, float scale, int window, int by_head, float *part, int part_tiles, int dtype,
                                      b200_stream_t stream) {
    B200_REQUIRE(ql && (qr || rot_dim == 0) && pool && ol && tiles && block_table, "latent_attention_tiles: null pointer");
    B200_REQUIRE(n_tiles >= 0 && heads > 0 && kv_rank > 0 && rot_dim >= 0 && window >= 0 && t_pad > 0, "latent_attention_tiles: bad shape");
    B200_REQUIRE(((uintptr_t)tiles & 15) == 0, "latent_attention_tiles: the tile list must be 16-byte aligned");
    B200_REQUIRE(!part || part_tiles >= n_tiles, "latent_attention_tiles: the partial-result scratch holds %d tiles, %d given", part_tiles, n_tiles);
    return launch_latent_attention_tiles(dtype, ql, qr, pool, sink, ol, tiles, n_tiles, block_table, max_pages_per_seq, t_pad, heads, kv_rank, rot_dim,
                                         scale, window, by_head, part, part_tiles, as_stream(stream));
}
}
