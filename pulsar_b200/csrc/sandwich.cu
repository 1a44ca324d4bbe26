// Memory-bound kernels of layers that also normalise a sublayer's output, and of the clamped gated unit.
//
//   post_norm_add    residual += rmsnorm(delta) * w_post  (the norm behind a sublayer, float32 sums, added into
//                    the float32 residual stream), and in the same pass, where the next norm is known,
//                    out = rmsnorm(residual) * w_next: one kernel between two sublayers instead of three.
//   clamped_glu      gate_up [N, 2I] (gate columns, then up columns) -> out [N, I]:
//                    g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1),
//                    float32 arithmetic, one rounding on store.
//   post_norm_add_bias   the same for layers whose sublayers read the stream itself: residual += rmsnorm(delta + bias) *
//                    w_post (bias optional: the bias of the projection that made delta), and out = the stream as it
//                    now is, in the activation dtype, for the sublayer that reads it next.  Without delta: out only.
//   glu_bias         gate_up [N, 2I] + bias [2I] -> out [N, I] with the gating of the fused products (limit, alpha,
//                    shift; SwiGLU is inf, 1, 0): the gated unit of a feed-forward whose projections have biases.
#include "common.cuh"

#include <stdint.h>

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

// The same with the row held in registers: 4 elements per thread and vector (VPT vectors per thread), one read of every
// input, 16-byte accesses of the float32 stream.  width % 4 == 0, 16-byte aligned rows.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename T, int VPT>
__global__ void post_norm_add_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ w_post,
                                         float eps_post, const float* __restrict__ w_next, float eps_next, T* __restrict__ out,
                                         int width) {
    pdl_wait();         // may have come onto the SMs while the product before it was ending: nothing is touched before that one is done
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * width;
    const T* del = delta + (size_t)r * width;
    float x[VPT][4];
    float ss = 0.0f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            load4(del + i, x[v]);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += x[v][e] * x[v][e];
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps_post);
    float ss2 = 0.0f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            float rv[4], wv[4];
            load4(res + i, rv);
            load4(w_post + i, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[v][e] = rv[e] + x[v][e] * inv * wv[e];
                ss2 += x[v][e] * x[v][e];
            }
            store4(res + i, x[v]);
        }
    }
    if (w_next == nullptr) return;              // uniform over the block
    const float inv2 = rsqrtf(block_sum(ss2, scratch) / (float)width + eps_next);
    T* o = out + (size_t)r * width;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            float wv[4], y[4];
            load4(w_next + i, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = x[v][e] * inv2 * wv[e];
            store4(o + i, y);
        }
    }
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

template <typename T>
__global__ void post_norm_add_bias_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ bias,
                                          const float* __restrict__ w_post, float eps_post, T* __restrict__ out, int width) {
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * width;
    if (delta != nullptr) {                       // uniform over the grid
        const T* del = delta + (size_t)r * width;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float d = to_float(del[i]) + (bias ? bias[i] : 0.0f);
            ss += d * d;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps_post);
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float d = to_float(del[i]) + (bias ? bias[i] : 0.0f);
            const float x = res[i] + d * inv * w_post[i];
            res[i] = x;
            if (out != nullptr) out[(size_t)r * width + i] = from_float<T>(x);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)r * width + i] = from_float<T>(res[i]);
}

// The same with the row in registers and 16-byte accesses (width % 4 == 0, 16-byte aligned rows, delta given).
template <typename T, int VPT>
__global__ void post_norm_add_bias_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta, const float* __restrict__ bias,
                                              const float* __restrict__ w_post, float eps_post, T* __restrict__ out, int width) {
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float* res = residual + (size_t)r * width;
    const T* del = delta + (size_t)r * width;
    float x[VPT][4];
    float ss = 0.0f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            load4(del + i, x[v]);
            if (bias != nullptr) {
                float b[4];
                load4(bias + i, b);
#pragma unroll
                for (int e = 0; e < 4; ++e) x[v][e] += b[e];
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += x[v][e] * x[v][e];
        }
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps_post);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * 4;
        if (i < width) {
            float rv[4], wv[4];
            load4(res + i, rv);
            load4(w_post + i, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) x[v][e] = rv[e] + x[v][e] * inv * wv[e];
            store4(res + i, x[v]);
            if (out != nullptr) store4(out + (size_t)r * width + i, x[v]);
        }
    }
}

template <typename TIn, typename T>
__global__ void glu_bias_kernel(const TIn* __restrict__ gate_up, const float* __restrict__ bias, T* __restrict__ out, size_t total,
                                const GatedInter p) {
    pdl_wait();
    const int inter = p.n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / inter, col = i % inter;
        const float g = to_float(gate_up[row * 2 * inter + col]) + (bias ? bias[col] : 0.0f);
        const float u = to_float(gate_up[row * 2 * inter + inter + col]) + (bias ? bias[inter + col] : 0.0f);
        out[i] = from_float<T>(gated(g, u, p));
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
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && width <= 8192 && aligned && (dtype == PB_F32 || dtype == PB_BF16)) {
        const int vecs = width / 4;
        const int vpt = vecs <= 1024 ? 1 : 2;
        const int threads = ((vecs + vpt - 1) / vpt + 31) / 32 * 32;
#define PB_POST(T, V) launch_pdl(post_norm_add_vec_kernel<T, V>, n, threads, 0, stream, residual, (const T*)delta, w_post, eps_post, w_next, eps_next, (T*)out, width)
        if (dtype == PB_F32) { if (vpt == 1) PB_POST(float, 1); else PB_POST(float, 2); }
        else { if (vpt == 1) PB_POST(__nv_bfloat16, 1); else PB_POST(__nv_bfloat16, 2); }
#undef PB_POST
        return launch_status();
    }
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

// residual [n, width] float32 += rmsnorm(delta + bias) * w_post, and out [n, width] (dtype) = residual where out is given;
// delta null: out = residual only (bias, w_post unused).
PB_EXPORT int pb_post_norm_add_bias(int dtype, float* residual, const void* delta, const float* bias, const float* w_post,
                                    float eps_post, void* out, int n, int width, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (width <= 0 || (delta == nullptr && out == nullptr) || (delta != nullptr && w_post == nullptr)) return PB_ERR_BAD_SIZE;
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)bias | (uintptr_t)w_post | (uintptr_t)out) & 15) == 0;
    if (delta != nullptr && width % 4 == 0 && width <= 8192 && aligned && (dtype == PB_F32 || dtype == PB_BF16)) {
        const int vecs = width / 4;
        const int vpt = vecs <= 1024 ? 1 : 2;
        const int threads = ((vecs + vpt - 1) / vpt + 31) / 32 * 32;
#define PB_POSTB(T, V) return launch_pdl(post_norm_add_bias_vec_kernel<T, V>, dim3(n), dim3(threads), 0, stream, residual, (const T*)delta, bias, \
                                         w_post, eps_post, (T*)out, width)
        if (dtype == PB_F32) { if (vpt == 1) PB_POSTB(float, 1); else PB_POSTB(float, 2); }
        else { if (vpt == 1) PB_POSTB(__nv_bfloat16, 1); else PB_POSTB(__nv_bfloat16, 2); }
#undef PB_POSTB
    }
    const int b = block_for(width);
    if (dtype == PB_F32)
        return launch_pdl(post_norm_add_bias_kernel<float>, dim3(n), dim3(b), 0, stream, residual, (const float*)delta, bias, w_post,
                          eps_post, (float*)out, width);
    if (dtype == PB_BF16)
        return launch_pdl(post_norm_add_bias_kernel<__nv_bfloat16>, dim3(n), dim3(b), 0, stream, residual, (const __nv_bfloat16*)delta,
                          bias, w_post, eps_post, (__nv_bfloat16*)out, width);
    return PB_ERR_BAD_DTYPE;
}

// out [n, inter] (dtype) = gated(gate + bias[:inter], up + bias[inter:]) with gate_up [n, 2 inter] (in_dtype: float32 or
// dtype); limit <= 0 means none.
PB_EXPORT int pb_glu_bias(int in_dtype, int dtype, const void* gate_up, const float* bias, void* out, int n, int inter, float limit,
                          float alpha, float shift, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (inter <= 0) return PB_ERR_BAD_SIZE;
    const size_t total = (size_t)n * inter;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const GatedInter p(inter, limit > 0.0f ? limit : __builtin_huge_valf(), alpha, shift);
#define PB_GLU(TI, T) return launch_pdl(glu_bias_kernel<TI, T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const TI*)gate_up, bias, \
                                        (T*)out, total, p)
    if (in_dtype == PB_F32 && dtype == PB_F32) PB_GLU(float, float);
    if (in_dtype == PB_F32 && dtype == PB_BF16) PB_GLU(float, __nv_bfloat16);
    if (in_dtype == PB_BF16 && dtype == PB_BF16) PB_GLU(__nv_bfloat16, __nv_bfloat16);
#undef PB_GLU
    return PB_ERR_BAD_DTYPE;
}
