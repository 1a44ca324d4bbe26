// Paged attention in its general form: keys and values of different widths, an optional
// distance bias per head, a sliding window and a chunk mask, float32 queries.
//
// What the kinds of attention that the head-size-specific kernels do not cover share:
//   * key rows `Dk` wide and value rows `Dv` wide, each with a row stride of its own, so that
//     the value may be a leading part of the cached key row (attention over a compressed
//     latent: key = [latent | rotated part], value = latent, one cached tensor);
//   * score = (q . k) * scale - slope[h] * (p - j) where `slopes` is given (a linear distance
//     bias; p the query's position, j the key's);
//   * visible keys lo .. p with lo the largest of 0, p - window + 1 (window > 0) and
//     floor(p / chunk) * chunk (chunk > 0; chunks are counted from position 0 of the sequence).
// Queries come in float32 (rotation and score are 32-bit arithmetic whatever the cache holds);
// scores, the running maximum, the sums and the output accumulate in float32 with expf.
//
// One block per (query token, query head); key tiles of 32 aligned to absolute key indices,
// tile i handled by warp i mod 4, warps combined in index order: the result at a position does
// not depend on how the tokens were cut into steps, on what else is in the batch or on which
// pages hold the keys.  Prompt portions and single decoded tokens take the same kernel.
//
// Layouts: q [N, Hq, Dk] float32; out [N, Hq, Dv] T; pools [pages, Hkv, page_size, stride] T;
// block_table [S, table_stride]; cu_q [S+1]; kv_len [S] (after this step); seq_of_token [N].
//
// Also here: the kernel that splits a fused projection row [q | k | v] of such widths into float32
// queries and the pages.
#include "common.cuh"

namespace {

using namespace pb;

constexpr int kWarps = 4;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void load16(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

struct GeneralShape {
    int Hq, Hkv, Dk, Dv, k_stride, v_stride, page_size, window, chunk, table_stride;
    int k_vec;          // leading key elements that 16-byte loads may take (0 when rows are not 16-byte aligned)
    float scale;
};

template <typename T, int ACC>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_general_kernel(const float* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                               T* __restrict__ out, const int* __restrict__ block_table, const int* __restrict__ cu_q,
                               const int* __restrict__ kv_len, const int* __restrict__ seq_of_token,
                               const float* __restrict__ slopes, const GeneralShape sh, const PoolBounds bounds) {
    extern __shared__ float smem[];
    const int Dk = sh.Dk, Dv = sh.Dv;
    float* q_s = smem;                         // [Dk] query times scale
    float* p_s = q_s + Dk;                     // [kWarps][32]
    float* m_s = p_s + kWarps * 32;            // [kWarps]
    float* l_s = m_s + kWarps;                 // [kWarps]
    float* acc_s = l_s + kWarps;               // [kWarps][Dv]

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = seq_of_token[t];
    const int q0 = cu_q[s], q1 = cu_q[s + 1];
    const int p = kv_len[s] - (q1 - q0) + (t - q0);
    int lo = 0;
    if (sh.window > 0 && p - sh.window + 1 > lo) lo = p - sh.window + 1;
    if (sh.chunk > 0 && (p / sh.chunk) * sh.chunk > lo) lo = (p / sh.chunk) * sh.chunk;
    const int g = h / (sh.Hq / sh.Hkv);
    const int* table = block_table + (size_t)s * sh.table_stride;
    const float slope = slopes ? slopes[h] : 0.0f;

    const float* qv = q + ((size_t)t * sh.Hq + h) * Dk;
    for (int i = threadIdx.x; i < Dk; i += blockDim.x) q_s[i] = qv[i] * sh.scale;
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.0f;

    const int first_tile = lo >> 5, last_tile = p >> 5;
    for (int tile = first_tile + warp; tile <= last_tile; tile += kWarps) {
        const int j = (tile << 5) + lane;
        const bool valid = j >= lo && j <= p;
        float sc = -INFINITY;
        if (valid) {
            int page = table[j / sh.page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* kr = k_pool + (((size_t)page * sh.Hkv + g) * sh.page_size + j % sh.page_size) * sh.k_stride;
            float dot = 0.0f;
            int d = 0;
            for (; d < sh.k_vec; d += Vec<T>::n) {
                float kf[Vec<T>::n];
                load16(kr + d, kf);
#pragma unroll
                for (int e = 0; e < Vec<T>::n; ++e) dot = fmaf(q_s[d + e], kf[e], dot);
            }
            for (; d < Dk; ++d) dot = fmaf(q_s[d], to_float(kr[d]), dot);
            sc = dot - slope * (float)(p - j);
        }
        const float m_new = fmaxf(m_run, warp_max(sc));      // finite: every tile in range has a visible key
        const float pv = valid ? expf(sc - m_new) : 0.0f;
        const float corr = expf(m_run - m_new);               // 0 on the first tile (m_run = -inf)
        l_run = l_run * corr + warp_sum(pv);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= corr;
        __syncwarp();
        p_s[warp * 32 + lane] = pv;
        __syncwarp();
        const int j0 = tile << 5;
        const int k_begin = (lo > j0) ? lo - j0 : 0;
        const int k_end = (p - j0 < 31) ? p - j0 : 31;
        for (int kk = k_begin; kk <= k_end; ++kk) {
            const int jj = j0 + kk;
            int page = table[jj / sh.page_size];
            if (!page_ok(page, bounds)) page = 0;
            const T* vr = v_pool + (((size_t)page * sh.Hkv + g) * sh.page_size + jj % sh.page_size) * sh.v_stride;
            const float pk = p_s[warp * 32 + kk];
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < Dv) acc[i] = fmaf(pk, to_float(vr[d]), acc[i]);
            }
        }
    }

    if (lane == 0) { m_s[warp] = m_run; l_s[warp] = l_run; }
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc_s[warp * Dv + d] = acc[i];
    }
    __syncthreads();
    float m_all = m_s[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) m_all = fmaxf(m_all, m_s[w]);
    float l_all = 0.0f;
    float f[kWarps];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { f[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - m_all); l_all += l_s[w] * f[w]; }
    T* ov = out + ((size_t)t * sh.Hq + h) * Dv;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) o += acc_s[w * Dv + d] * f[w];
        ov[d] = from_float<T>(o / l_all);
    }
}

template <typename T, int ACC>
int launch_general(const float* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, const int* cu_q,
                   const int* kv_len, const int* seq_of_token, const float* slopes, int n_tokens, const GeneralShape& sh,
                   cudaStream_t stream) {
    const size_t smem = sizeof(float) * (sh.Dk + kWarps * 32 + 2 * kWarps + (size_t)kWarps * sh.Dv);
    dim3 grid(n_tokens, sh.Hq);
    paged_attention_general_kernel<T, ACC><<<grid, kWarps * 32, smem, stream>>>(q, (const T*)k_pool, (const T*)v_pool, (T*)out,
        block_table, cu_q, kv_len, seq_of_token, slopes, sh, pb::pool_bounds_now());
    return launch_status();
}

template <typename T>
int dispatch_general(const float* q, const void* k_pool, const void* v_pool, void* out, const int* block_table, const int* cu_q,
                     const int* kv_len, const int* seq_of_token, const float* slopes, int n_tokens, GeneralShape sh,
                     cudaStream_t stream) {
    const bool aligned = ((uintptr_t)k_pool % 16 == 0) && ((size_t)sh.k_stride * sizeof(T)) % 16 == 0;
    sh.k_vec = aligned ? sh.Dk - sh.Dk % Vec<T>::n : 0;
#define PB_GENERAL(A) return launch_general<T, A>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, n_tokens, sh, stream)
    if (sh.Dv <= 64) PB_GENERAL(2);
    if (sh.Dv <= 128) PB_GENERAL(4);
    if (sh.Dv <= 256) PB_GENERAL(8);
    if (sh.Dv <= 512) PB_GENERAL(16);
    PB_GENERAL(32);
#undef PB_GENERAL
}

// One warp per (token, head) of the fused projection row [q: Hq*Dk | k: Hkv*Dk | v: Hkv*Dv]:
// queries to float32 [N, Hq, Dk], keys and values into the pages of the token's slot.
template <typename T>
__global__ void qkv_split_write_kernel(const T* __restrict__ qkv, float* __restrict__ q_out, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, const int* __restrict__ slots, int Hq, int Hkv, int Dk, int Dv,
                                       int page_size, const PoolBounds bounds) {
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= Hq + 2 * Hkv) return;
    const size_t row = (size_t)Hq * Dk + (size_t)Hkv * (Dk + Dv);
    const T* base = qkv + (size_t)t * row;
    if (head < Hq) {
        const T* src = base + (size_t)head * Dk;
        float* dst = q_out + ((size_t)t * Hq + head) * Dk;
        for (int i = lane; i < Dk; i += 32) dst[i] = to_float(src[i]);
        return;
    }
    const int slot = slots[t];
    if (slot < 0 || !slot_ok(slot, page_size, bounds)) return;
    const bool is_k = head < Hq + Hkv;
    const int kvh = is_k ? head - Hq : head - Hq - Hkv;
    const int D = is_k ? Dk : Dv;
    const T* src = base + (size_t)Hq * Dk + (is_k ? (size_t)kvh * Dk : (size_t)Hkv * Dk + (size_t)kvh * Dv);
    T* dst = (is_k ? k_pool : v_pool) + (((size_t)(slot / page_size) * Hkv + kvh) * page_size + slot % page_size) * D;
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
}

}  // namespace

PB_EXPORT int pb_paged_attention_general(int dtype, const float* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                                         const int* seq_of_token, const float* slopes, int n_tokens, int Hq, int Hkv, int Dk,
                                         int Dv, int k_stride, int v_stride, int page_size, float scale, int window, int chunk,
                                         cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Dk <= 0 || Dv <= 0 || Dk > 4096 || Dv > 1024 || Hkv <= 0 || Hq <= 0 || Hq % Hkv || page_size <= 0 || k_stride < Dk ||
        v_stride < Dv || window < 0 || chunk < 0)
        return PB_ERR_BAD_SIZE;
    if (Hq > 65535) return PB_ERR_TOO_LARGE;
    GeneralShape sh{Hq, Hkv, Dk, Dv, k_stride, v_stride, page_size, window, chunk, table_stride, 0, scale};
    if (dtype == PB_F32)
        return dispatch_general<float>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, n_tokens, sh, stream);
    if (dtype == PB_BF16)
        return dispatch_general<__nv_bfloat16>(q, k_pool, v_pool, out, block_table, cu_q, kv_len, seq_of_token, slopes, n_tokens, sh,
                                               stream);
    return PB_ERR_BAD_DTYPE;
}

PB_EXPORT int pb_qkv_split_write(int dtype, const void* qkv, float* q_out, void* k_pool, void* v_pool, const int* slots,
                                 int n_tokens, int Hq, int Hkv, int Dk, int Dv, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (Hq <= 0 || Hkv < 0 || Dk <= 0 || Dv <= 0 || page_size <= 0) return PB_ERR_BAD_SIZE;
    const int heads = Hq + 2 * Hkv;
    dim3 grid(n_tokens, (heads + 3) / 4);
    if (dtype == PB_F32)
        qkv_split_write_kernel<float><<<grid, 128, 0, stream>>>((const float*)qkv, q_out, (float*)k_pool, (float*)v_pool, slots, Hq,
                                                                Hkv, Dk, Dv, page_size, pb::pool_bounds_now());
    else if (dtype == PB_BF16)
        qkv_split_write_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)qkv, q_out, (__nv_bfloat16*)k_pool,
                                                                        (__nv_bfloat16*)v_pool, slots, Hq, Hkv, Dk, Dv, page_size,
                                                                        pb::pool_bounds_now());
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}
