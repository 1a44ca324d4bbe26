// Helpers of attention over a compressed latent (one cached row per token: [latent | rotated key part]).
//
//   heads_linear     out[n, h, :] = W[h]^T a[n, h, :] (W[h] stored [K, M]) for every head h: the per-head products that
//                    stand in for expanding the latent into keys and values.  With the key
//                    expansion W_uk the query side takes q_abs[h] = W_uk[h]^T q_plain[h]
//                    (so that q_plain . (W_uk[h] c) = q_abs[h] . c), with the value expansion W_uv
//                    the output side takes W_uv[h] (sum_j p_j c_j).  float32 accumulation.  A few tokens: a
//                    block takes 8 tokens x 32 outputs, four slices of K in ascending k each, added in slice
//                    order (enough blocks to fill the GPU).  Many tokens: 8 tokens x 128 outputs, K whole.
//                    Optionally multiplies by sigmoid(gate[n, h, :]) (an output gate) in float32.
//   latent_prepare   per token: RMS norm of the latent part of the down projection (float32),
//                    rotation of the shared key part at the token's position, both written to
//                    the token's cache slot (and, where asked, to contiguous rows for the expanded form);
//                    rotation of every head's rotated query part into its float32 query row
//                    ([q_abs | q_rot], or [q_plain | q_rot] for the expanded form).
//   latent_expand_keys, sigmoid_gate: the expanded form's key rows [plain | shared rotated part], and its output gate.
// The rotation pairs neighbours: (x[2i], x[2i+1]) turns by the angle of table column i; dimensions
// beyond the rotated ones pass unchanged.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kTok = 8;

// Many tokens: one thread per output over the whole of K, 128 outputs a block.
template <typename T, typename TO>
__global__ void __launch_bounds__(128)
heads_linear_wide_kernel(const T* __restrict__ a, long a_tok, int a_head, const T* __restrict__ w, TO* __restrict__ out, long o_tok,
                         int o_head, const T* __restrict__ gate, long g_tok, int N, int M, int K) {
    extern __shared__ __align__(16) float smem[];  // [kTok][KP], KP = K rounded up to a multiple of 4 (zeros behind K)
    float* a_s = smem;
    const int KP = (K + 3) & ~3;
    const int n0 = blockIdx.x * kTok, h = blockIdx.y;
    const int nt = min(kTok, N - n0);
    for (int i = threadIdx.x; i < kTok * KP; i += blockDim.x) {
        const int tt = i / KP, k = i % KP;
        a_s[i] = (tt < nt && k < K) ? to_float(a[(size_t)(n0 + tt) * a_tok + (size_t)h * a_head + k]) : 0.0f;
    }
    __syncthreads();
    const int m = blockIdx.z * blockDim.x + threadIdx.x;
    if (m >= M) return;
    const T* wh = w + (size_t)h * K * M + m;
    float acc[kTok];
#pragma unroll
    for (int tt = 0; tt < kTok; ++tt) acc[tt] = 0.0f;
    for (int k = 0; k < KP; k += 4) {
        float wv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) wv[e] = (k + e < K) ? to_float(wh[(size_t)(k + e) * M]) : 0.0f;
#pragma unroll
        for (int tt = 0; tt < kTok; ++tt) {
            const float4 av = *reinterpret_cast<const float4*>(a_s + tt * KP + k);
            acc[tt] = fmaf(av.x, wv[0], acc[tt]);
            acc[tt] = fmaf(av.y, wv[1], acc[tt]);
            acc[tt] = fmaf(av.z, wv[2], acc[tt]);
            acc[tt] = fmaf(av.w, wv[3], acc[tt]);
        }
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

constexpr int kSlices = 4;      // a block's 128 threads: 32 outputs x 4 slices of K
constexpr int kBatch = 16;      // weights a thread asks for before it uses the first

template <typename T, typename TO>
__global__ void __launch_bounds__(128)
heads_linear_kernel(const T* __restrict__ a, long a_tok, int a_head, const T* __restrict__ w, TO* __restrict__ out, long o_tok,
                    int o_head, const T* __restrict__ gate, long g_tok, int N, int M, int K) {
    pdl_wait();         // may have come onto the SMs while the product before it was ending: nothing is touched before that one is done
    extern __shared__ __align__(16) float smem[];
    const int KS = (((K + kSlices - 1) / kSlices) + kBatch - 1) / kBatch * kBatch;      // k's per slice, a multiple of kBatch
    const int KP = KS * kSlices;
    float* a_s = smem;                             // [kTok][KP], zeros behind K
    float* r_s = a_s + kTok * KP;                  // [kSlices][kTok][32] partial sums
    const int n0 = blockIdx.x * kTok, h = blockIdx.y;
    const int nt = min(kTok, N - n0);
    for (int i = threadIdx.x; i < kTok * KP; i += blockDim.x) {
        const int tt = i / KP, k = i % KP;
        a_s[i] = (tt < nt && k < K) ? to_float(a[(size_t)(n0 + tt) * a_tok + (size_t)h * a_head + k]) : 0.0f;
    }
    __syncthreads();
    const int mx = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int m = blockIdx.z * 32 + mx;
    const bool live = m < M;
    const T* wh = w + (size_t)h * K * M + (live ? m : 0);       // [K, M]: neighbouring threads read neighbouring weights
    float acc[kTok];
#pragma unroll
    for (int tt = 0; tt < kTok; ++tt) acc[tt] = 0.0f;
    const int k0 = slice * KS;
    for (int k = k0; k < k0 + KS; k += kBatch) {
        float wv[kBatch];                          // a batch of weights on their way at once
#pragma unroll
        for (int e = 0; e < kBatch; ++e) wv[e] = (live && k + e < K) ? to_float(wh[(size_t)(k + e) * M]) : 0.0f;
#pragma unroll
        for (int e = 0; e < kBatch; e += 4) {
#pragma unroll
            for (int tt = 0; tt < kTok; ++tt) {
                const float4 av = *reinterpret_cast<const float4*>(a_s + tt * KP + k + e);
                acc[tt] = fmaf(av.x, wv[e], acc[tt]);
                acc[tt] = fmaf(av.y, wv[e + 1], acc[tt]);
                acc[tt] = fmaf(av.z, wv[e + 2], acc[tt]);
                acc[tt] = fmaf(av.w, wv[e + 3], acc[tt]);
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < kTok; ++tt) r_s[(slice * kTok + tt) * 32 + mx] = acc[tt];
    __syncthreads();
    // the slices are added in their order by one thread per (token, output)
    for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
        const int tt = i >> 5, x = i & 31, mm = blockIdx.z * 32 + x;
        if (mm >= M) continue;
        float v = 0.0f;
#pragma unroll
        for (int sl = 0; sl < kSlices; ++sl) v += r_s[(sl * kTok + tt) * 32 + x];
        if (gate) {
            const float gv = to_float(gate[(size_t)(n0 + tt) * g_tok + (size_t)h * M + mm]);
            v *= 1.0f / (1.0f + expf(-gv));
        }
        out[(size_t)(n0 + tt) * o_tok + (size_t)h * o_head + mm] = from_float<TO>(v);
    }
}

struct PrepareShape {
    int H, dim, rot_dim, rot_dims, rank, page_size;
    int q_row, q_off, copy_plain;       // rows of q_out are q_row wide; the rotated part goes to q_off; plain dimensions are copied to the front or not
    long q_tok, down_tok;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ q, const T* __restrict__ down, const float* __restrict__ norm_w,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ slots,
                      T* __restrict__ pool, float* __restrict__ q_out, T* __restrict__ latent_out, T* __restrict__ rot_out,
                      const PrepareShape sh, const PoolBounds bounds) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int rank = sh.rank, rot_dim = sh.rot_dim, half = sh.rot_dims >> 1;
    const float* ct = cos_t + (size_t)t * half;
    const float* st = sin_t + (size_t)t * half;
    if (down != nullptr) {                      // uniform over the block
        const T* x = down + (size_t)t * sh.down_tok;
        float ss = 0.0f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_float(x[i]); ss += v * v; }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)rank + sh.eps);
        const int slot = slots[t];
        const bool cached = slot >= 0 && slot_ok(slot, sh.page_size, bounds);
        T* dst = pool + (size_t)(cached ? slot : 0) * (rank + rot_dim);   // [pages, 1, page, rank + rot_dim]: slot = page * page_size + offset
        T* lat = latent_out ? latent_out + (size_t)t * rank : nullptr;
        T* rot = rot_out ? rot_out + (size_t)t * rot_dim : nullptr;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const T v = from_float<T>(to_float(x[i]) * inv * norm_w[i]);
            if (cached) dst[i] = v;
            if (lat) lat[i] = v;
        }
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float u = to_float(x[rank + 2 * i]), v = to_float(x[rank + 2 * i + 1]);
            const T a = from_float<T>(u * ct[i] - v * st[i]), b = from_float<T>(v * ct[i] + u * st[i]);
            if (cached) { dst[rank + 2 * i] = a; dst[rank + 2 * i + 1] = b; }
            if (rot) { rot[2 * i] = a; rot[2 * i + 1] = b; }
        }
        for (int i = sh.rot_dims + threadIdx.x; i < rot_dim; i += blockDim.x) {
            if (cached) dst[rank + i] = x[rank + i];
            if (rot) rot[i] = x[rank + i];
        }
    }
    const int per_head = sh.dim + rot_dim, H = sh.H;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        const T* src = q + (size_t)t * sh.q_tok + (size_t)h * per_head + sh.dim;
        float* dst = q_out + ((size_t)t * H + h) * sh.q_row + sh.q_off;
        const float u = to_float(src[2 * j]), v = to_float(src[2 * j + 1]);
        dst[2 * j] = u * ct[j] - v * st[j];
        dst[2 * j + 1] = v * ct[j] + u * st[j];
    }
    const int rest = rot_dim - sh.rot_dims;
    for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
        const int h = i / rest, j = sh.rot_dims + i % rest;
        q_out[((size_t)t * H + h) * sh.q_row + sh.q_off + j] = to_float(q[(size_t)t * sh.q_tok + (size_t)h * per_head + sh.dim + j]);
    }
    if (sh.copy_plain) {
        for (int i = threadIdx.x; i < H * sh.dim; i += blockDim.x) {
            const int h = i / sh.dim, j = i % sh.dim;
            q_out[((size_t)t * H + h) * sh.q_row + j] = to_float(q[(size_t)t * sh.q_tok + (size_t)h * per_head + j]);
        }
    }
}

// keys[n, h, :] = [plain[n, h, :dim] | shared[n, :rot_dim]]: every head's expanded plain key beside the rotated part all heads share.
template <typename T>
__global__ void latent_expand_keys_kernel(const T* __restrict__ plain, const T* __restrict__ shared, T* __restrict__ keys, int H,
                                          int dim, int rot_dim) {
    const int t = blockIdx.x, row = dim + rot_dim;
    for (int i = threadIdx.x; i < H * row; i += blockDim.x) {
        const int h = i / row, j = i % row;
        keys[(size_t)t * H * row + i] = j < dim ? plain[((size_t)t * H + h) * dim + j] : shared[(size_t)t * rot_dim + j - dim];
    }
}

// x[n, c] *= sigmoid(gate[n, c]) with float32 arithmetic; gate rows g_tok apart.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, long g_tok, int width, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / width, c = i % width;
        x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-to_float(gate[n * g_tok + c]))));
    }
}

template <typename T, typename TO>
int launch_heads(const void* a, long a_tok, int a_head, const void* w, void* out, long o_tok, int o_head, const void* gate,
                 long g_tok, int N, int H, int M, int K, cudaStream_t stream) {
    if (N > 2 * kTok) {         // enough token tiles to fill the GPU without cutting K
        dim3 wide((N + kTok - 1) / kTok, H, (M + 127) / 128);
        heads_linear_wide_kernel<T, TO><<<wide, 128, sizeof(float) * kTok * ((K + 3) & ~3), stream>>>(
            (const T*)a, a_tok, a_head, (const T*)w, (TO*)out, o_tok, o_head, (const T*)gate, g_tok, N, M, K);
        return launch_status();
    }
    const int ks = (((K + kSlices - 1) / kSlices) + kBatch - 1) / kBatch * kBatch;
    dim3 grid((N + kTok - 1) / kTok, H, (M + 31) / 32);
    launch_pdl(heads_linear_kernel<T, TO>, grid, 128, sizeof(float) * kTok * (ks * kSlices + kSlices * 32), stream, (const T*)a, a_tok, a_head, (const T*)w, (TO*)out,
                                                                                 o_tok, o_head, (const T*)gate, g_tok, N, M, K);
    return launch_status();
}

}  // namespace

// out[n, h, m] = sum_k a[n, h, k] * w[h, k, m]  (* sigmoid(gate[n, h * M + m]) where a gate is given).
// a: element (n, h, k) at n * a_tok + h * a_head + k; out likewise with o_tok, o_head; w contiguous [H, K, M].
// dtype: of a, w and gate; out_dtype: of out (float32, or the same as dtype).
PB_EXPORT int pb_heads_linear(int dtype, int out_dtype, const void* a, long a_tok, int a_head, const void* w, void* out, long o_tok,
                              int o_head, const void* gate, long g_tok, int N, int H, int M, int K, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || M <= 0 || K <= 0 || K > 1024 || (M + 31) / 32 > 65535) return PB_ERR_BAD_SIZE;
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
// pool [pages, 1, page_size, rank + rot_dim].  q_out float32 [N, H, q_row]: every head's rotated part, turned, at q_off;
// with copy_plain its plain dimensions at 0.  latent_out [N, rank] / rot_out [N, rot_dim] (may be null): what went to the cache.
PB_EXPORT int pb_latent_prepare(int dtype, const void* q, long q_tok, const void* down, long down_tok, const float* norm_w,
                                float eps, const float* cos_t, const float* sin_t, const int* slots, void* pool, float* q_out,
                                int q_row, int q_off, int copy_plain, void* latent_out, void* rot_out, int N, int H, int dim,
                                int rot_dim, int rot_dims, int rank, int page_size, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || dim < 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 || rank <= 0 || page_size <= 0 ||
        q_off < 0 || q_off + rot_dim > q_row || (copy_plain && dim > q_off))
        return PB_ERR_BAD_SIZE;
    if (down != nullptr && (norm_w == nullptr || slots == nullptr || pool == nullptr)) return PB_ERR_BAD_SIZE;
    const PrepareShape sh{H, dim, rot_dim, rot_dims, rank, page_size, q_row, q_off, copy_plain, q_tok, down_tok, eps};
    if (dtype == PB_F32)
        latent_prepare_kernel<float><<<N, 128, 0, stream>>>((const float*)q, (const float*)down, norm_w, cos_t, sin_t, slots,
                                                            (float*)pool, q_out, (float*)latent_out, (float*)rot_out, sh,
                                                            pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<N, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)down, norm_w, cos_t,
                                                                    sin_t, slots, (__nv_bfloat16*)pool, q_out,
                                                                    (__nv_bfloat16*)latent_out, (__nv_bfloat16*)rot_out, sh,
                                                                    pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_latent_expand_keys(int dtype, const void* plain, const void* shared, void* keys, int N, int H, int dim, int rot_dim,
                                    cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || dim < 0 || rot_dim < 0 || dim + rot_dim <= 0) return PB_ERR_BAD_SIZE;
    if (dtype == PB_F32)
        latent_expand_keys_kernel<float><<<N, 256, 0, stream>>>((const float*)plain, (const float*)shared, (float*)keys, H, dim, rot_dim);
    else if (dtype == PB_BF16)
        latent_expand_keys_kernel<__nv_bfloat16><<<N, 256, 0, stream>>>((const __nv_bfloat16*)plain, (const __nv_bfloat16*)shared,
                                                                        (__nv_bfloat16*)keys, H, dim, rot_dim);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

PB_EXPORT int pb_sigmoid_gate(int dtype, void* x, const void* gate, long g_tok, int N, int width, cudaStream_t stream) {
    if (N <= 0 || width <= 0) return 0;
    const size_t total = (size_t)N * width;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PB_F32) sigmoid_gate_kernel<float><<<(int)blocks, 256, 0, stream>>>((float*)x, (const float*)gate, g_tok, width, total);
    else if (dtype == PB_BF16)
        sigmoid_gate_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)gate, g_tok, width, total);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
