// Helpers of attention over a compressed latent (one cached row per token: [latent | rotated key part]).
//
//   heads_linear     out[n, h, :] = W[h] a[n, h, :] for every head h: the per-head products that
//                    stand in for expanding the latent into keys and values.  With the key
//                    expansion W_uk the query side takes q_abs[h] = W_uk[h]^T q_plain[h]
//                    (so that q_plain . (W_uk[h] c) = q_abs[h] . c), with the value expansion W_uv
//                    the output side takes W_uv[h] (sum_j p_j c_j).  float32 accumulation in
//                    ascending k, one thread per output, the tokens of a tile share the weights.
//                    Optionally multiplies by sigmoid(gate[n, h, :]) (an output gate) in float32.
//   latent_prepare   per token: RMS norm of the latent part of the down projection (float32),
//                    rotation of the shared key part at the token's position, both written to
//                    the token's cache slot; rotation of every head's rotated query part into
//                    the tail of its float32 query row [q_abs | q_rot].
// The rotation pairs neighbours: (x[2i], x[2i+1]) turns by the angle of table column i; dimensions
// beyond the rotated ones pass unchanged.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kTok = 8;

template <typename T, typename TO>
__global__ void __launch_bounds__(128)
heads_linear_kernel(const T* __restrict__ a, long a_tok, int a_head, const T* __restrict__ w, TO* __restrict__ out, long o_tok,
                    int o_head, const T* __restrict__ gate, long g_tok, int N, int M, int K) {
    extern __shared__ float a_s[];                 // [kTok][K]
    const int n0 = blockIdx.x * kTok, h = blockIdx.y;
    const int nt = min(kTok, N - n0);
    for (int i = threadIdx.x; i < kTok * K; i += blockDim.x) {
        const int tt = i / K, k = i % K;
        a_s[i] = tt < nt ? to_float(a[(size_t)(n0 + tt) * a_tok + (size_t)h * a_head + k]) : 0.0f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * M * K;
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const T* wr = wh + (size_t)m * K;
        float acc[kTok];
#pragma unroll
        for (int tt = 0; tt < kTok; ++tt) acc[tt] = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float wv = to_float(wr[k]);
#pragma unroll
            for (int tt = 0; tt < kTok; ++tt) acc[tt] = fmaf(a_s[tt * K + k], wv, acc[tt]);
        }
        for (int tt = 0; tt < nt; ++tt) {
            float v = acc[tt];
            if (gate) {
                const float gv = to_float(gate[(size_t)(n0 + tt) * g_tok + (size_t)h * M + m]);
                v *= 1.0f / (1.0f + expf(-gv));
            }
            out[(size_t)(n0 + tt) * o_tok + (size_t)h * o_head + m] = from_float<TO>(v);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ q, long q_tok, const T* __restrict__ down, long down_tok,
                      const float* __restrict__ norm_w, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, const int* __restrict__ slots, T* __restrict__ pool,
                      float* __restrict__ q_full, int H, int dim, int rot_dim, int rot_dims, int rank, int page_size,
                      const PoolBounds bounds) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int half = rot_dims >> 1;
    const float* ct = cos_t + (size_t)t * half;
    const float* st = sin_t + (size_t)t * half;
    if (down != nullptr) {                      // uniform over the block
        const T* x = down + (size_t)t * down_tok;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_float(x[i]); ss += v * v; }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)rank + eps);
        const int slot = slots[t];
        if (slot >= 0 && slot_ok(slot, page_size, bounds)) {
            T* dst = pool + (size_t)slot * (rank + rot_dim);        // [pages, 1, page, rank + rot_dim]: slot = page * page_size + offset
            for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(x[i]) * inv * norm_w[i]);
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float u = to_float(x[rank + 2 * i]), v = to_float(x[rank + 2 * i + 1]);
                dst[rank + 2 * i] = from_float<T>(u * ct[i] - v * st[i]);
                dst[rank + 2 * i + 1] = from_float<T>(v * ct[i] + u * st[i]);
            }
            for (int i = rot_dims + threadIdx.x; i < rot_dim; i += blockDim.x) dst[rank + i] = x[rank + i];
        }
    }
    const int per_head = dim + rot_dim;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        const T* src = q + (size_t)t * q_tok + (size_t)h * per_head + dim;
        float* dst = q_full + ((size_t)t * H + h) * (rank + rot_dim) + rank;
        const float u = to_float(src[2 * j]), v = to_float(src[2 * j + 1]);
        dst[2 * j] = u * ct[j] - v * st[j];
        dst[2 * j + 1] = v * ct[j] + u * st[j];
    }
    const int rest = rot_dim - rot_dims;
    for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
        const int h = i / rest, j = rot_dims + i % rest;
        q_full[((size_t)t * H + h) * (rank + rot_dim) + rank + j] = to_float(q[(size_t)t * q_tok + (size_t)h * per_head + dim + j]);
    }
}

template <typename T, typename TO>
int launch_heads(const void* a, long a_tok, int a_head, const void* w, void* out, long o_tok, int o_head, const void* gate,
                 long g_tok, int N, int H, int M, int K, cudaStream_t stream) {
    dim3 grid((N + kTok - 1) / kTok, H);
    heads_linear_kernel<T, TO><<<grid, 128, sizeof(float) * kTok * K, stream>>>((const T*)a, a_tok, a_head, (const T*)w, (TO*)out,
                                                                                 o_tok, o_head, (const T*)gate, g_tok, N, M, K);
    return launch_status();
}

}  // namespace

// out[n, h, m] = sum_k a[n, h, k] * w[h, m, k]  (* sigmoid(gate[n, h * M + m]) where a gate is given).
// a: element (n, h, k) at n * a_tok + h * a_head + k; out likewise with o_tok, o_head; w contiguous [H, M, K].
// dtype: of a, w and gate; out_dtype: of out (float32, or the same as dtype).
PB_EXPORT int pb_heads_linear(int dtype, int out_dtype, const void* a, long a_tok, int a_head, const void* w, void* out, long o_tok,
                              int o_head, const void* gate, long g_tok, int N, int H, int M, int K, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || M <= 0 || K <= 0 || K > 1024) return PB_ERR_BAD_SIZE;
    if (H > 65535) return PB_ERR_TOO_LARGE;
    if (dtype == PB_F32 && out_dtype == PB_F32)
        return launch_heads<float, float>(a, a_tok, a_head, w, out, o_tok, o_head, gate, g_tok, N, H, M, K, stream);
    if (dtype == PB_BF16 && out_dtype == PB_F32)
        return launch_heads<__nv_bfloat16, float>(a, a_tok, a_head, w, out, o_tok, o_head, gate, g_tok, N, H, M, K, stream);
    if (dtype == PB_BF16 && out_dtype == PB_BF16)
        return launch_heads<__nv_bfloat16, __nv_bfloat16>(a, a_tok, a_head, w, out, o_tok, o_head, gate, g_tok, N, H, M, K, stream);
    return PB_ERR_BAD_DTYPE;
}

// q: the projected query rows, head h at q + n * q_tok + h * (dim + rot_dim), its rotated part behind `dim` plain
// dimensions.  down (may be null: the layer borrows another layer's cache): rows of rank + rot_dim at n * down_tok.
// pool [pages, 1, page_size, rank + rot_dim]; q_full float32 [N, H, rank + rot_dim] (only the tail is written).
PB_EXPORT int pb_latent_prepare(int dtype, const void* q, long q_tok, const void* down, long down_tok, const float* norm_w,
                                float eps, const float* cos_t, const float* sin_t, const int* slots, void* pool, float* q_full,
                                int N, int H, int dim, int rot_dim, int rot_dims, int rank, int page_size, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || dim < 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 || rank <= 0 || page_size <= 0)
        return PB_ERR_BAD_SIZE;
    if (down != nullptr && (norm_w == nullptr || slots == nullptr || pool == nullptr)) return PB_ERR_BAD_SIZE;
    if (dtype == PB_F32)
        latent_prepare_kernel<float><<<N, 128, 0, stream>>>((const float*)q, q_tok, (const float*)down, down_tok, norm_w, eps, cos_t,
                                                            sin_t, slots, (float*)pool, q_full, H, dim, rot_dim, rot_dims, rank,
                                                            page_size, pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<N, 128, 0, stream>>>((const __nv_bfloat16*)q, q_tok, (const __nv_bfloat16*)down,
                                                                    down_tok, norm_w, eps, cos_t, sin_t, slots, (__nv_bfloat16*)pool,
                                                                    q_full, H, dim, rot_dim, rot_dims, rank, page_size,
                                                                    pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
