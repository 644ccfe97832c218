// moe.cu -- mixture-of-experts feed-forward for ragged token batches.
//   route:   scores = sigmoid(router logits) (fp32); the `top` largest are chosen, their scores ARE the weights (no renormalisation);
//            a separate sigmoid gate scales the shared expert.
//   plan:    the (token, choice) pairs are grouped by expert; every expert's rows are padded to whole tiles of kMoeTileM rows so that a
//            tile of the grouped GEMM belongs to exactly one expert.  Done on the device: the host never learns the counts, it launches
//            the worst-case number of tiles and the surplus CTAs leave at once.
//   gather:  row <- T(weight * x[token])  -- the weight multiplies the expert's input, which matters for a non-linear expert;
//   grouped GEMM (x2): up with the activation in the epilogue, then down.
// The sum over a token's experts, the shared expert and the post-norm are one kernel of the engine (hybrid.cu).
#include "hybrid_ops.cuh"

namespace b200 {

__device__ __forceinline__ float act_apply(float v, int act) {
    if (act == B200_ACT_RELU2) {
        const float r = fmaxf(v, 0.0f);
        return r * r;
    }
    if (act == B200_ACT_SILU) return v / (1.0f + expf(-v));
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    return 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
}

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

// one CTA.  Shared: count[E] | offset[E+1] | cursor[E]
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int *__restrict__ sel_expert, const float *__restrict__ sel_weight, int *__restrict__ row_token, float *__restrict__ row_weight,
                int *__restrict__ tile_expert, int *__restrict__ pair_row, int *__restrict__ n_tiles, int pairs, int experts, int top) {
    extern __shared__ int si[];
    int *count = si, *offset = si + experts, *cursor = offset + experts + 1;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0, cursor[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[sel_expert[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            offset[e] = at;
            const int tiles = (count[e] + kMoeTileM - 1) / kMoeTileM;
            for (int i = 0; i < tiles; ++i) tile_expert[at / kMoeTileM + i] = e;
            at += tiles * kMoeTileM;
        }
        offset[experts] = at;
        *n_tiles = at / kMoeTileM;
    }
    __syncthreads();
    const int rows = offset[experts];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) row_token[r] = -1, row_weight[r] = 0.0f;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = sel_expert[p];
        const int r = offset[e] + atomicAdd(&cursor[e], 1);
        row_token[r] = p / top;
        row_weight[r] = sel_weight[p];
        pair_row[p] = r;
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const float *__restrict__ x, const int *__restrict__ row_token, const float *__restrict__ row_weight, T *__restrict__ xg,
                  const int *__restrict__ n_tiles, int width) {
    const int r = blockIdx.x;
    if (r >= *n_tiles * kMoeTileM) return;
    const int t = row_token[r];
    const float w = row_weight[r];
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        xg[(size_t)r * width + c] = Elem<T>::from_f(t >= 0 ? w * x[(size_t)t * width + c] : 0.0f);
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

template <typename T>
__global__ void activation_kernel(T *__restrict__ x, size_t n, int act) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = Elem<T>::from_f(act_apply(Elem<T>::to_f(x[i]), act));
}

int launch_moe_route_sigmoid(const float *logits, int ld, int *sel_expert, float *sel_weight, float *shared_gate, int tokens,
                             int experts, int top, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    moe_route_sigmoid_kernel<<<(tokens + 3) / 4, 128, 0, st>>>(logits, ld, sel_expert, sel_weight, shared_gate, tokens, experts, top);
    return cuda_status("moe_route launch");
}

int launch_moe_plan(const int *sel_expert, const float *sel_weight, int *row_token, float *row_weight, int *tile_expert, int *pair_row,
                    int *n_tiles, int tokens, int experts, int top, int max_rows, cudaStream_t st) {
    (void)max_rows;
    moe_plan_kernel<<<1, 1024, (size_t)(3 * experts + 1) * sizeof(int), st>>>(sel_expert, sel_weight, row_token, row_weight, tile_expert,
                                                                             pair_row, n_tiles, tokens * top, experts, top);
    return cuda_status("moe_plan launch");
}

int launch_moe_gather(int dtype, const float *x, const int *row_token, const float *row_weight, void *xg, const int *n_tiles,
                      int max_rows, int width, cudaStream_t st) {
    if (max_rows == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, { moe_gather_kernel<T><<<max_rows, 128, 0, st>>>(x, row_token, row_weight, (T *)xg, n_tiles, width); });
    return cuda_status("moe_gather launch");
}

int launch_moe_grouped_gemm(int dtype, const void *a, const void *w, void *c, const int *tile_expert, const int *n_tiles, int max_tiles,
                            int N, int K, int act, cudaStream_t st) {
    if (max_tiles == 0) return B200_OK;
    const dim3 grid((N + kGT - 1) / kGT, max_tiles);
    B200_DISPATCH_DTYPE(dtype, {
        moe_grouped_gemm_kernel<T><<<grid, 256, 0, st>>>((const T *)a, (const T *)w, (T *)c, tile_expert, n_tiles, N, K, act);
    });
    return cuda_status("moe_grouped_gemm launch");
}

int launch_activation(int dtype, void *x, size_t n, int act, cudaStream_t st) {
    if (n == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, { activation_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((T *)x, n, act); });
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
