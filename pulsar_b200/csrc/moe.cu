// A mixture of gated experts: the router, and the experts' products for steps of a few tokens.
//
//   moe_route      z = W_r h in float32 (W_r float32 [E, width]; h in the activation dtype), s = sigmoid(z), the `top`
//                  largest s per token (ties: the lower index), weights s * scale, or with `renormalize` s / sum of the
//                  chosen s * scale.  ids int32 [N, top] in descending order of s, weights float32 [N, top].
//   moe_gate_up    for every (token, chosen expert): g = W_gate[e] h, u = W_up[e] h (float32 sums), the gated unit
//                  out = g' * sigmoid(alpha * g') * (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit),
//                  one rounding on store: act [N * top, ff].  Weights [E, 2 ff, width]: an expert's gate rows, then
//                  its up rows.
//   moe_down       out[n] = add[n] + sum over the chosen experts, in the order of ids, of weight * (W_down[e] act[n, slot]);
//                  float32 sums, one rounding on store.  Weights [E, width, ff].  `add` (optional): what a shared
//                  expert contributed.
// A warp owns one output element and walks the contraction in a fixed order, so a token's result does not depend on
// what else is in the step.  These kernels read an expert's weights once per token that chose it: they are for steps
// of a few tokens (and for the float32 engine); larger steps sort the tokens by expert and take the grouped product.
#include "common.cuh"

namespace {

using namespace pb;

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, int* __restrict__ ids,
                                 float* __restrict__ weights, int width, int n_experts, int top, float scale, int renormalize) {
    pdl_wait();
    extern __shared__ float smem[];
    float* x = smem;                         // [width]
    float* s = smem + width;                 // [n_experts]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[i] = to_float(h[(size_t)t * width + i]);
    __syncthreads();
    for (int e = warp; e < n_experts; e += warps) {
        const float* w = router + (size_t)e * width;
        float z = 0.0f;
        for (int i = lane; i < width; i += 32) z = fmaf(w[i], x[i], z);
        z = warp_sum(z);
        if (lane == 0) s[e] = 1.0f / (1.0f + expf(-z));
    }
    __syncthreads();
    if (warp != 0) return;
    float total = 0.0f;
    for (int c = 0; c < top; ++c) {
        // the largest score left; among equals the lowest index
        float best = -1.0f;
        int arg = n_experts;
        for (int e = lane; e < n_experts; e += 32)
            if (s[e] > best) { best = s[e]; arg = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (lane == 0) {
            ids[(size_t)t * top + c] = arg;
            weights[(size_t)t * top + c] = best;
            s[arg] = -2.0f;                  // taken
        }
        total += best;
        __syncwarp();
    }
    if (lane == 0) {
        const float f = renormalize ? scale / total : scale;
        for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] *= f;
    }
}

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float acc = 0.0f;
    for (int i = lane; i < n; i += 32) acc = fmaf(to_float(w[i]), x[i], acc);
    return warp_sum(acc);
}

template <typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gate_up, const int* __restrict__ ids,
                                   T* __restrict__ act, int width, int ff, int top, const GatedInter p) {
    pdl_wait();
    extern __shared__ float x[];             // [width]
    const int pair = blockIdx.x, t = pair / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[i] = to_float(h[(size_t)t * width + i]);
    __syncthreads();
    const int e = ids[pair];
    const T* w = w_gate_up + (size_t)e * 2 * ff * width;
    for (int j = blockIdx.y * warps + warp; j < ff; j += gridDim.y * warps) {
        const float g = dot_row(w + (size_t)j * width, x, width, lane);
        const float u = dot_row(w + (size_t)(ff + j) * width, x, width, lane);
        if (lane == 0) act[(size_t)pair * ff + j] = from_float<T>(gated(g, u, p));
    }
}

template <typename T>
__global__ void moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int* __restrict__ ids,
                                const float* __restrict__ weights, const T* __restrict__ add, T* __restrict__ out, int width,
                                int ff, int top) {
    pdl_wait();
    extern __shared__ float y[];             // [top][ff]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) y[i] = to_float(act[(size_t)t * top * ff + i]);
    __syncthreads();
    for (int c = blockIdx.y * warps + warp; c < width; c += gridDim.y * warps) {
        float sum = add ? to_float(add[(size_t)t * width + c]) : 0.0f;
        for (int slot = 0; slot < top; ++slot) {
            const int e = ids[(size_t)t * top + slot];
            const float d = dot_row(w_down + ((size_t)e * width + c) * ff, y + (size_t)slot * ff, ff, lane);
            sum = fmaf(weights[(size_t)t * top + slot], d, sum);
        }
        if (lane == 0) out[(size_t)t * width + c] = from_float<T>(sum);
    }
}

}  // namespace

PB_EXPORT int pb_moe_route(int dtype, const void* h, const float* router, int* ids, float* weights, int n, int width, int n_experts,
                           int top, float scale, int renormalize, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || n_experts <= 0 || top <= 0 || top > n_experts) return PB_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * ((size_t)width + n_experts);
    if (smem > 48 * 1024) return PB_ERR_TOO_LARGE;
    if (dtype == PB_F32)
        return launch_pdl(moe_route_kernel<float>, dim3(n), dim3(128), smem, stream, (const float*)h, router, ids, weights, width,
                          n_experts, top, scale, renormalize);
    if (dtype == PB_BF16)
        return launch_pdl(moe_route_kernel<__nv_bfloat16>, dim3(n), dim3(128), smem, stream, (const __nv_bfloat16*)h, router, ids,
                          weights, width, n_experts, top, scale, renormalize);
    return PB_ERR_BAD_DTYPE;
}

PB_EXPORT int pb_moe_gate_up(int dtype, const void* h, const void* w_gate_up, const int* ids, void* act, int n, int width, int ff,
                             int top, float limit, float alpha, float shift, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return PB_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * (size_t)width;
    if (smem > 48 * 1024) return PB_ERR_TOO_LARGE;
    const int warps = 8;
    int by = (ff + warps - 1) / warps;
    if (by > 64) by = 64;
    const GatedInter p(ff, limit > 0.0f ? limit : __builtin_huge_valf(), alpha, shift);
    dim3 grid(n * top, by);
    if (dtype == PB_F32)
        return launch_pdl(moe_gate_up_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)h, (const float*)w_gate_up, ids,
                          (float*)act, width, ff, top, p);
    if (dtype == PB_BF16)
        return launch_pdl(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)h,
                          (const __nv_bfloat16*)w_gate_up, ids, (__nv_bfloat16*)act, width, ff, top, p);
    return PB_ERR_BAD_DTYPE;
}

PB_EXPORT int pb_moe_down(int dtype, const void* act, const void* w_down, const int* ids, const float* weights, const void* add,
                          void* out, int n, int width, int ff, int top, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || ff <= 0 || top <= 0) return PB_ERR_BAD_SIZE;
    const size_t smem = sizeof(float) * (size_t)top * ff;
    if (smem > 48 * 1024) return PB_ERR_TOO_LARGE;
    const int warps = 8;
    int by = (width + warps - 1) / warps;
    if (by > 64) by = 64;
    dim3 grid(n, by);
    if (dtype == PB_F32)
        return launch_pdl(moe_down_kernel<float>, grid, dim3(warps * 32), smem, stream, (const float*)act, (const float*)w_down, ids,
                          weights, (const float*)add, (float*)out, width, ff, top);
    if (dtype == PB_BF16)
        return launch_pdl(moe_down_kernel<__nv_bfloat16>, grid, dim3(warps * 32), smem, stream, (const __nv_bfloat16*)act,
                          (const __nv_bfloat16*)w_down, ids, weights, (const __nv_bfloat16*)add, (__nv_bfloat16*)out, width, ff, top);
    return PB_ERR_BAD_DTYPE;
}
