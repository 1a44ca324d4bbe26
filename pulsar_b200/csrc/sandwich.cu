// Memory-bound kernels of layers that also normalise a sublayer's output, and of the clamped gated unit.
//
//   post_norm_add    residual += rmsnorm(delta) * w_post  (the norm behind a sublayer, float32 sums, added into
//                    the float32 residual stream), and in the same pass, where the next norm is known,
//                    out = rmsnorm(residual) * w_next: one kernel between two sublayers instead of three.
//   clamped_glu      gate_up [N, 2I] (gate columns, then up columns) -> out [N, I]:
//                    g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1),
//                    float32 arithmetic, one rounding on store.
#include "common.cuh"

namespace {

using namespace pb;

template <typename T>
__global__ void post_norm_add_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ w_post,
                                     float eps_post, const float* __restrict__ w_next, float eps_next, T* __restrict__ out,
                                     int width) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * width;
    const T* del = delta + (size_t)r * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = to_float(del[i]); ss += d * d; }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps_post);
    float ss2 = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = res[i] + to_float(del[i]) * inv * w_post[i];
        res[i] = x;
        ss2 += x * x;
    }
    if (w_next == nullptr) return;              // uniform over the block
    const float inv2 = rsqrtf(block_sum(ss2, scratch) / (float)width + eps_next);
    T* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_float<T>(res[i] * inv2 * w_next[i]);   // own writes
}

template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total, float limit,
                                   float alpha) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / inter, col = i % inter;
        const float g = fminf(to_float(gate_up[row * 2 * inter + col]), limit);
        const float u = fminf(fmaxf(to_float(gate_up[row * 2 * inter + inter + col]), -limit), limit);
        out[i] = from_float<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

int block_for(int width) {
    int b = 32;
    while (b < 1024 && b * 4 < width) b <<= 1;
    return b;
}

}  // namespace

// residual [n, width] float32 += rmsnorm(delta) * w_post; with w_next also out [n, width] = rmsnorm(residual) * w_next.
PB_EXPORT int pb_post_norm_add(int dtype, float* residual, const void* delta, const float* w_post, float eps_post,
                               const float* w_next, float eps_next, void* out, int n, int width, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || (w_next != nullptr && out == nullptr)) return PB_ERR_BAD_SIZE;
    const int b = block_for(width);
    if (dtype == PB_F32)
        post_norm_add_kernel<float><<<n, b, 0, stream>>>(residual, (const float*)delta, w_post, eps_post, w_next, eps_next,
                                                         (float*)out, width);
    else if (dtype == PB_BF16)
        post_norm_add_kernel<__nv_bfloat16><<<n, b, 0, stream>>>(residual, (const __nv_bfloat16*)delta, w_post, eps_post, w_next,
                                                                 eps_next, (__nv_bfloat16*)out, width);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_clamped_glu(int dtype, const void* gate_up, void* out, int n, int inter, float limit, float alpha,
                             cudaStream_t stream) {
    if (n <= 0) return 0;
    if (inter <= 0) return PB_ERR_BAD_SIZE;
    const size_t total = (size_t)n * inter;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PB_F32)
        clamped_glu_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, total, limit, alpha);
    else if (dtype == PB_BF16)
        clamped_glu_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter,
                                                                           total, limit, alpha);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
