// The recurrent mixer of the selective state-space kind: a short causal convolution per channel and
// the selective scan, both over a ragged batch of prompt portions and single decoded tokens, with
// the state of every sequence in a slot of a float32 arena.
//
//   causal_conv_silu   x[t, c] = silu(bias[c] + sum_tau taps[c, tau] * in(p - (T-1) + tau, c)); the
//                      last column of the taps weighs the current token.  Inputs before the
//                      portion's start come from the slot's tail (the last T-1 inputs of the
//                      sequence, zeros at its very start).
//   selective_scan     dt = softplus(W_dt r + dt_bias) (r the dt part of the input-dependent
//                      projection; the product is done here, in float32, dt_rank terms per
//                      channel), A = -exp(A_log),
//                        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n
//                        y_c = (sum_n S[c, n] C_n + D_c x_c) * silu(z_c)
//                      token after token for each sequence; S lives in registers between the
//                      tokens of a portion and in the slot between steps.  When a portion is
//                      done the kernel also moves the slot's convolution tail on.
// Everything that enters the recurrence (dt, softplus, the decay and its exponential, the state,
// the sums over the state) is float32; x, z, B, C and r arrive in the activation dtype.
//
// Slot layout (float32): [inner, state] scan state, then [inner, T-1] convolution tail.
//
// Thread layout of the scan: G lanes per channel share the channel's state (lane l holds states
// l, l + G, ...; at most 8 each) and its dt weights (at most 32 each); a block of 128 threads takes
// 128 / G channels of one sequence; the tokens are staged through shared memory 16 at a time.
#include "common.cuh"

namespace {

using namespace pb;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const T* __restrict__ in, long in_tok, const float* __restrict__ taps, const float* __restrict__ bias,
                        const float* __restrict__ arena, long slot_stride, long tail_offset, const int* __restrict__ cu_q,
                        const int* __restrict__ seq_of_token, const int* __restrict__ state_slots, T* __restrict__ out,
                        int channels, int n_taps) {
    pdl_wait();         // may have come onto the SMs while the product before it was ending: nothing is touched before that one is done
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int s = seq_of_token[t];
    const int i = t - cu_q[s];                          // index within the portion
    const float* tail = arena + (size_t)state_slots[s] * slot_stride + tail_offset + (size_t)c * (n_taps - 1);
    float acc = bias[c];
    for (int tau = 0; tau < n_taps; ++tau) {
        const int back = n_taps - 1 - tau;
        const float v = (i - back >= 0) ? to_float(in[(size_t)(t - back) * in_tok + c]) : tail[n_taps - 1 + i - back];
        acc = fmaf(taps[(size_t)c * n_taps + tau], v, acc);
    }
    out[(size_t)t * channels + c] = from_float<T>(silu_f(acc));
}

constexpr int kStage = 16;          // tokens staged per round
constexpr int kStagePrompt = 32;    // the same in the kernel for portions
constexpr int kBatchTokens = 8;     // tokens whose state-independent work that kernel does side by side
constexpr int kStatesPerLane = 8;
constexpr int kDtPerLane = 32;

struct ScanShape {
    int inner, n_state, dt_rank, n_taps;
    long slot_stride, tail_offset, xz_tok, proj_tok;
};

template <typename T, int G>
__global__ void __launch_bounds__(128)
selective_scan_kernel(const T* __restrict__ x, const T* __restrict__ xz, const T* __restrict__ proj, const T* __restrict__ w_dt,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      float* __restrict__ arena, T* __restrict__ y, const int* __restrict__ cu_q,
                      const int* __restrict__ state_slots, const ScanShape sh) {
    pdl_wait();         // may have come onto the SMs while the product before it was ending: nothing is touched before that one is done
    constexpr int CH = 128 / G;
    extern __shared__ float smem[];
    const int S = sh.n_state, R = sh.dt_rank, inner = sh.inner;
    float* bc_s = smem;                               // [kStage][2 * S]
    float* r_s = bc_s + kStage * 2 * S;               // [kStage][R]
    float* x_s = r_s + kStage * R;                    // [kStage][CH]
    float* z_s = x_s + kStage * CH;                   // [kStage][CH]

    const int seq = blockIdx.x;
    const int group = threadIdx.x / G, gl = threadIdx.x % G;
    const int c0 = blockIdx.y * CH;
    const int c = c0 + group;
    const bool live = c < inner;
    const int q0 = cu_q[seq], q_len = cu_q[seq + 1] - q0;
    float* slot = arena + (size_t)state_slots[seq] * sh.slot_stride;

    float a[kStatesPerLane], st[kStatesPerLane], wd[kDtPerLane];
#pragma unroll
    for (int j = 0; j < kStatesPerLane; ++j) {
        const int n = gl + G * j;
        const bool on = live && n < S;
        a[j] = on ? -expf(a_log[(size_t)c * S + n]) : 0.0f;
        st[j] = on ? slot[(size_t)c * S + n] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < kDtPerLane; ++j) {
        const int r = gl + G * j;
        wd[j] = (live && r < R) ? to_float(w_dt[(size_t)c * R + r]) : 0.0f;
    }
    const float bias = live ? dt_bias[c] : 0.0f;
    const float skip = live ? d_skip[c] : 0.0f;

    for (int base = 0; base < q_len; base += kStage) {
        const int nt = min(kStage, q_len - base);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 2 * S; i += blockDim.x) {
            const int tt = i / (2 * S), k = i % (2 * S);
            bc_s[tt * 2 * S + k] = to_float(proj[(size_t)(q0 + base + tt) * sh.proj_tok + R + k]);
        }
        for (int i = threadIdx.x; i < nt * R; i += blockDim.x) {
            const int tt = i / R, k = i % R;
            r_s[tt * R + k] = to_float(proj[(size_t)(q0 + base + tt) * sh.proj_tok + k]);
        }
        for (int i = threadIdx.x; i < nt * CH; i += blockDim.x) {
            const int tt = i / CH, k = i % CH;
            const bool on = c0 + k < inner;
            const size_t row = (size_t)(q0 + base + tt);
            x_s[tt * CH + k] = on ? to_float(x[row * inner + c0 + k]) : 0.0f;
            z_s[tt * CH + k] = on ? to_float(xz[row * sh.xz_tok + inner + c0 + k]) : 0.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float dt = 0.0f;
#pragma unroll
            for (int j = 0; j < kDtPerLane; ++j) {
                const int r = gl + G * j;
                if (r < R) dt = fmaf(wd[j], r_s[tt * R + r], dt);
            }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) dt += __shfl_xor_sync(0xffffffffu, dt, o);
            dt = softplus_f(dt + bias);
            const float xv = x_s[tt * CH + group];
            const float dx = dt * xv;
            const float* bt = bc_s + tt * 2 * S;
            float part = 0.0f;
#pragma unroll
            for (int j = 0; j < kStatesPerLane; ++j) {
                const int n = gl + G * j;
                if (n < S) {
                    st[j] = fmaf(expf(dt * a[j]), st[j], dx * bt[n]);
                    part = fmaf(st[j], bt[S + n], part);
                }
            }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (live && gl == 0)
                y[(size_t)(q0 + base + tt) * inner + c] = from_float<T>((part + skip * xv) * silu_f(z_s[tt * CH + group]));
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < kStatesPerLane; ++j) {
        const int n = gl + G * j;
        if (n < S) slot[(size_t)c * S + n] = st[j];
    }
    if (gl == 0) {
        // the tail moves on: its entry k becomes the convolution's input at index q_len - (T-1) + k of this portion, or, where
        // the portion is shorter than the tail, the old entry k + q_len (read before anything at or above it is written)
        float* tail = slot + sh.tail_offset + (size_t)c * (sh.n_taps - 1);
        for (int k = 0; k < sh.n_taps - 1; ++k) {
            const int j = q_len - (sh.n_taps - 1) + k;
            tail[k] = j >= 0 ? to_float(xz[(size_t)(q0 + j) * sh.xz_tok + c]) : tail[k + q_len];
        }
    }
}

// The scan for prompt portions: the step sizes before their bias and softplus come from a product of their own
// (dt_pre [N, inner] float32), and the tokens of a staged round are taken eight at a time: what does not depend on the
// state (softplus, the decays' exponentials) is computed for the eight first, so that only the multiply-adds of the
// state chain from token to token, and the eight sums over the state are reduced side by side.  SPL: states per lane.
template <typename T, int G, int SPL>
__global__ void __launch_bounds__(128)
selective_scan_prompt_kernel(const T* __restrict__ x, const T* __restrict__ xz, const T* __restrict__ bc, long bc_tok,
                             const float* __restrict__ dt_pre, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                             const float* __restrict__ d_skip, float* __restrict__ arena, T* __restrict__ y,
                             const int* __restrict__ cu_q, const int* __restrict__ state_slots, const ScanShape sh) {
    constexpr int CH = 128 / G;
    constexpr int U = kBatchTokens;
    extern __shared__ float smem[];
    const int S = sh.n_state, inner = sh.inner;
    float* bc_s = smem;                               // [kStagePrompt][2 * S]
    float* x_s = bc_s + kStagePrompt * 2 * S;               // [kStagePrompt][CH]
    float* z_s = x_s + kStagePrompt * CH;                   // [kStagePrompt][CH]
    float* dt_s = z_s + kStagePrompt * CH;                  // [kStagePrompt][CH]

    const int seq = blockIdx.x;
    const int group = threadIdx.x / G, gl = threadIdx.x % G;
    const int c0 = blockIdx.y * CH;
    const int c = c0 + group;
    const bool live = c < inner;
    const int q0 = cu_q[seq], q_len = cu_q[seq + 1] - q0;
    float* slot = arena + (size_t)state_slots[seq] * sh.slot_stride;

    float a[SPL], st[SPL];
#pragma unroll
    for (int j = 0; j < SPL; ++j) {
        const int n = gl + G * j;
        const bool on = live && n < S;
        a[j] = on ? -expf(a_log[(size_t)c * S + n]) : 0.0f;
        st[j] = on ? slot[(size_t)c * S + n] : 0.0f;
    }
    const float bias = live ? dt_bias[c] : 0.0f;
    const float skip = live ? d_skip[c] : 0.0f;

    for (int base = 0; base < q_len; base += kStagePrompt) {
        const int nt = min(kStagePrompt, q_len - base);
        __syncthreads();
        for (int i = threadIdx.x; i < kStagePrompt * 2 * S; i += blockDim.x) {
            const int tt = i / (2 * S), k = i % (2 * S);
            bc_s[i] = tt < nt ? to_float(bc[(size_t)(q0 + base + tt) * bc_tok + k]) : 0.0f;
        }
        for (int i = threadIdx.x; i < kStagePrompt * CH; i += blockDim.x) {
            const int tt = i / CH, k = i % CH;
            const bool on = tt < nt && c0 + k < inner;
            const size_t row = (size_t)(q0 + base + (on ? tt : 0));
            x_s[i] = on ? to_float(x[row * inner + c0 + k]) : 0.0f;
            z_s[i] = on ? to_float(xz[row * sh.xz_tok + inner + c0 + k]) : 0.0f;
            dt_s[i] = on ? dt_pre[row * inner + c0 + k] : 0.0f;
        }
        __syncthreads();
        for (int t0 = 0; t0 < nt; t0 += U) {
            float dx[U], da[U][SPL], part[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float dt = softplus_f(dt_s[(t0 + u) * CH + group] + bias);
                dx[u] = dt * x_s[(t0 + u) * CH + group];
#pragma unroll
                for (int j = 0; j < SPL; ++j) da[u][j] = expf(dt * a[j]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* bt = bc_s + (t0 + u) * 2 * S;
                const bool in = t0 + u < nt;                       // the rows behind the round's end hold zeros and must not move the state
                float p = 0.0f;
#pragma unroll
                for (int j = 0; j < SPL; ++j) {
                    const int n = gl + G * j;
                    if (n < S) {
                        const float next = fmaf(da[u][j], st[j], dx[u] * bt[n]);
                        st[j] = in ? next : st[j];
                        p = fmaf(next, bt[S + n], p);
                    }
                }
                part[u] = p;
            }
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < U; ++u) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
            if (live && gl < U && t0 + gl < nt) {
                float mine = part[0];
#pragma unroll
                for (int u = 1; u < U; ++u) mine = (gl == u) ? part[u] : mine;
                const int tt = t0 + gl;
                y[(size_t)(q0 + base + tt) * inner + c] =
                    from_float<T>((mine + skip * x_s[tt * CH + group]) * silu_f(z_s[tt * CH + group]));
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int j = 0; j < SPL; ++j) {
        const int n = gl + G * j;
        if (n < S) slot[(size_t)c * S + n] = st[j];
    }
    if (gl == 0) {
        float* tail = slot + sh.tail_offset + (size_t)c * (sh.n_taps - 1);
        for (int k = 0; k < sh.n_taps - 1; ++k) {
            const int j = q_len - (sh.n_taps - 1) + k;
            tail[k] = j >= 0 ? to_float(xz[(size_t)(q0 + j) * sh.xz_tok + c]) : tail[k + q_len];
        }
    }
}

template <typename T, int G, int SPL>
int launch_scan_prompt(const void* x, const void* xz, const void* bc, long bc_tok, const float* dt_pre, const float* dt_bias,
                       const float* a_log, const float* d_skip, float* arena, void* y, const int* cu_q, const int* state_slots,
                       int n_seqs, const ScanShape& sh, cudaStream_t stream) {
    constexpr int CH = 128 / G;
    const size_t smem = sizeof(float) * kStagePrompt * (2 * sh.n_state + 3 * CH);
    dim3 grid(n_seqs, (sh.inner + CH - 1) / CH);
    selective_scan_prompt_kernel<T, G, SPL><<<grid, 128, smem, stream>>>((const T*)x, (const T*)xz, (const T*)bc, bc_tok, dt_pre, dt_bias,
                                                                         a_log, d_skip, arena, (T*)y, cu_q, state_slots, sh);
    return launch_status();
}

// The scan for long portions, parallel over tokens.  For one channel and one state the recurrence S_t = a_t S_(t-1) + b_t
// (a_t = exp(dt_t A), b_t = dt_t x_t B_t) composes: a run of tokens acts on the state as S -> P S + Q with P the product of
// its a's and Q its own contribution.  A warp takes one channel and 256 tokens at a time: each lane walks its 8 consecutive
// tokens to get (P, Q) of its run, the 32 runs are combined by a prefix scan over the lanes (five shuffle steps), each
// lane takes the state that enters its run (the carried state of the span before, through the prefix of the lanes before
// it) and walks its 8 tokens again to accumulate y_t += S_t C_t.  The states are taken one after the other, so a lane keeps
// 8 step sizes, 8 inputs, 8 decays, 8 contributions and 8 outputs in registers.  A block of eight warps takes eight
// neighbouring channels and shares the staged B and C rows of the span.  Tokens behind a portion's end enter as dt = 0
// (a = 1, b = 0: they leave the state alone).  Shared-memory rows hold the span's tokens in the order [token in run][lane]
// (one more word than 256 per row), so that lanes read neighbouring words and the staging writes hit different banks.
constexpr int kSpan = 256, kRun = 8, kSpanRow = kSpan + 1, kChunkChannels = 8;

template <typename T>
__global__ void __launch_bounds__(256)
selective_scan_chunked_kernel(const T* __restrict__ x, const T* __restrict__ xz, const T* __restrict__ bc, long bc_tok,
                              const float* __restrict__ dt_pre, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                              const float* __restrict__ d_skip, float* __restrict__ arena, T* __restrict__ y,
                              const int* __restrict__ cu_q, const int* __restrict__ state_slots, const ScanShape sh) {
    extern __shared__ float smem[];
    const int S = sh.n_state, inner = sh.inner;
    float* bc_s = smem;                                      // [2 S][kSpanRow]
    float* x_s = bc_s + 2 * S * kSpanRow;                    // [8][kSpanRow]
    float* z_s = x_s + kChunkChannels * kSpanRow;
    float* dt_s = z_s + kChunkChannels * kSpanRow;
    float* y_s = dt_s + kChunkChannels * kSpanRow;           // [8][kSpanRow]
    float* a_s = y_s + kChunkChannels * kSpanRow;            // [8][S] decay rates A = -exp(A_log)
    float* carry_s = a_s + kChunkChannels * S;               // [8][S] the state between spans

    const int seq = blockIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c0 = blockIdx.y * kChunkChannels;
    const int c = c0 + w;
    const bool live = c < inner;
    const int q0 = cu_q[seq], q_len = cu_q[seq + 1] - q0;
    float* slot = arena + (size_t)state_slots[seq] * sh.slot_stride;
    for (int n = lane; n < S; n += 32) {
        a_s[w * S + n] = live ? -expf(a_log[(size_t)c * S + n]) : 0.0f;
        carry_s[w * S + n] = live ? slot[(size_t)c * S + n] : 0.0f;
    }
    const float bias = live ? dt_bias[c] : 0.0f;
    const float skip = live ? d_skip[c] : 0.0f;

    for (int base = 0; base < q_len; base += kSpan) {
        const int nt = min(kSpan, q_len - base);
        __syncthreads();                                     // the span before is done with (and a_s, carry_s are written)
        for (int i = threadIdx.x; i < kSpan * 2 * S; i += blockDim.x) {
            const int tt = i / (2 * S), k = i % (2 * S);
            const int at = (tt % kRun) * 32 + tt / kRun;     // [token in run][lane]
            bc_s[k * kSpanRow + at] = tt < nt ? to_float(bc[(size_t)(q0 + base + tt) * bc_tok + k]) : 0.0f;
        }
        for (int i = threadIdx.x; i < kSpan * kChunkChannels; i += blockDim.x) {
            const int tt = i / kChunkChannels, j = i % kChunkChannels;
            const int at = (tt % kRun) * 32 + tt / kRun;
            const bool on = tt < nt && c0 + j < inner;
            const size_t row = (size_t)(q0 + base + (on ? tt : 0));
            x_s[j * kSpanRow + at] = on ? to_float(x[row * inner + c0 + j]) : 0.0f;
            z_s[j * kSpanRow + at] = on ? to_float(xz[row * sh.xz_tok + inner + c0 + j]) : 0.0f;
            dt_s[j * kSpanRow + at] = on ? dt_pre[row * inner + c0 + j] : 0.0f;
        }
        __syncthreads();
        float dt[kRun], dx[kRun], acc[kRun];
#pragma unroll
        for (int k = 0; k < kRun; ++k) {
            const bool on = lane * kRun + k < nt;
            dt[k] = on ? softplus_f(dt_s[w * kSpanRow + k * 32 + lane] + bias) : 0.0f;     // 0: the token leaves the state alone
            dx[k] = dt[k] * x_s[w * kSpanRow + k * 32 + lane];
            acc[k] = 0.0f;
        }
        for (int n = 0; n < S; ++n) {
            const float rate = a_s[w * S + n];
            const float* bn = bc_s + n * kSpanRow + lane;
            const float* cn = bc_s + (S + n) * kSpanRow + lane;
            float a[kRun], b[kRun];
            float P = 1.0f, Q = 0.0f;
#pragma unroll
            for (int k = 0; k < kRun; ++k) {
                a[k] = expf(dt[k] * rate);
                b[k] = dx[k] * bn[k * 32];
                Q = fmaf(a[k], Q, b[k]);
                P *= a[k];
            }
            // inclusive prefix over the lanes: (P, Q) of all runs up to and including this lane's
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float Pp = __shfl_up_sync(0xffffffffu, P, o), Qp = __shfl_up_sync(0xffffffffu, Q, o);
                if (lane >= o) { Q = fmaf(P, Qp, Q); P *= Pp; }
            }
            const float carry = carry_s[w * S + n];
            float Pe = __shfl_up_sync(0xffffffffu, P, 1), Qe = __shfl_up_sync(0xffffffffu, Q, 1);
            if (lane == 0) { Pe = 1.0f; Qe = 0.0f; }
            float st = fmaf(Pe, carry, Qe);                  // the state that enters this lane's run
#pragma unroll
            for (int k = 0; k < kRun; ++k) {
                st = fmaf(a[k], st, b[k]);
                acc[k] = fmaf(st, cn[k * 32], acc[k]);
            }
            const float P_all = __shfl_sync(0xffffffffu, P, 31), Q_all = __shfl_sync(0xffffffffu, Q, 31);
            __syncwarp();                                    // every lane has read the carry
            if (lane == 0) carry_s[w * S + n] = fmaf(P_all, carry, Q_all);
        }
#pragma unroll
        for (int k = 0; k < kRun; ++k) {
            const int at = k * 32 + lane;
            y_s[w * kSpanRow + at] = (acc[k] + skip * x_s[w * kSpanRow + at]) * silu_f(z_s[w * kSpanRow + at]);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * kChunkChannels; i += blockDim.x) {
            const int tt = i / kChunkChannels, j = i % kChunkChannels;
            if (c0 + j < inner)
                y[(size_t)(q0 + base + tt) * inner + c0 + j] = from_float<T>(y_s[j * kSpanRow + (tt % kRun) * 32 + tt / kRun]);
        }
    }
    __syncwarp();
    if (!live) return;
    for (int n = lane; n < S; n += 32) slot[(size_t)c * S + n] = carry_s[w * S + n];
    if (lane == 0) {
        float* tail = slot + sh.tail_offset + (size_t)c * (sh.n_taps - 1);
        for (int k = 0; k < sh.n_taps - 1; ++k) {
            const int j = q_len - (sh.n_taps - 1) + k;
            tail[k] = j >= 0 ? to_float(xz[(size_t)(q0 + j) * sh.xz_tok + c]) : tail[k + q_len];
        }
    }
}

size_t chunked_smem(int n_state) {
    return sizeof(float) * ((size_t)(2 * n_state + 4 * kChunkChannels) * kSpanRow + 2 * kChunkChannels * n_state);
}

template <typename T>
int launch_scan_chunked(const void* x, const void* xz, const void* bc, long bc_tok, const float* dt_pre, const float* dt_bias,
                        const float* a_log, const float* d_skip, float* arena, void* y, const int* cu_q, const int* state_slots,
                        int n_seqs, const ScanShape& sh, cudaStream_t stream) {
    const size_t smem = chunked_smem(sh.n_state);
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(selective_scan_chunked_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid(n_seqs, (sh.inner + kChunkChannels - 1) / kChunkChannels);
    selective_scan_chunked_kernel<T><<<grid, 256, smem, stream>>>((const T*)x, (const T*)xz, (const T*)bc, bc_tok, dt_pre, dt_bias, a_log,
                                                                  d_skip, arena, (T*)y, cu_q, state_slots, sh);
    return launch_status();
}

template <typename T>
int dispatch_scan_prompt(const void* x, const void* xz, const void* bc, long bc_tok, const float* dt_pre, const float* dt_bias,
                         const float* a_log, const float* d_skip, float* arena, void* y, const int* cu_q, const int* state_slots,
                         int n_seqs, const ScanShape& sh, cudaStream_t stream) {
#define PB_SCAN(G, SPL) return launch_scan_prompt<T, G, SPL>(x, xz, bc, bc_tok, dt_pre, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh, stream)
    const int S = sh.n_state;
    if (S <= 8) PB_SCAN(8, 1);
    if (S <= 16) PB_SCAN(8, 2);
    if (S <= 32) PB_SCAN(8, 4);
    if (S <= 64) PB_SCAN(8, 8);
    if (S <= 128) PB_SCAN(32, 4);
    PB_SCAN(32, 8);
#undef PB_SCAN
}

template <typename T, int G>
int launch_scan(const void* x, const void* xz, const void* proj, const void* w_dt, const float* dt_bias, const float* a_log,
                const float* d_skip, float* arena, void* y, const int* cu_q, const int* state_slots, int n_seqs,
                const ScanShape& sh, cudaStream_t stream) {
    constexpr int CH = 128 / G;
    const size_t smem = sizeof(float) * kStage * (2 * sh.n_state + sh.dt_rank + 2 * CH);
    dim3 grid(n_seqs, (sh.inner + CH - 1) / CH);
    launch_pdl(selective_scan_kernel<T, G>, grid, 128, smem, stream, (const T*)x, (const T*)xz, (const T*)proj, (const T*)w_dt, dt_bias,
                                                             a_log, d_skip, arena, (T*)y, cu_q, state_slots, sh);
    return launch_status();
}

template <typename T>
int dispatch_scan(const void* x, const void* xz, const void* proj, const void* w_dt, const float* dt_bias, const float* a_log,
                  const float* d_skip, float* arena, void* y, const int* cu_q, const int* state_slots, int n_seqs,
                  const ScanShape& sh, cudaStream_t stream) {
    if (sh.n_state <= 8 * kStatesPerLane && sh.dt_rank <= 8 * kDtPerLane)
        return launch_scan<T, 8>(x, xz, proj, w_dt, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh, stream);
    return launch_scan<T, 32>(x, xz, proj, w_dt, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh, stream);
}

}  // namespace

// in: rows of the input projection, channel c of token t at in + t * in_tok + c.  out [N, channels].
// arena: float32, slot s at arena + s * slot_stride, its convolution tail [channels, taps - 1] at tail_offset.
PB_EXPORT int pb_causal_conv_silu(int dtype, const void* in, long in_tok, const float* taps, const float* bias, const float* arena,
                                  long slot_stride, long tail_offset, const int* cu_q, const int* seq_of_token,
                                  const int* state_slots, void* out, int n_tokens, int channels, int n_taps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (channels <= 0 || n_taps < 1) return PB_ERR_BAD_SIZE;
    dim3 grid(n_tokens, (channels + 255) / 256);
    if (grid.y > 65535) return PB_ERR_TOO_LARGE;
    if (dtype == PB_F32)
        launch_pdl(causal_conv_silu_kernel<float>, grid, 256, 0, stream, (const float*)in, in_tok, taps, bias, arena, slot_stride, tail_offset,
                                                                 cu_q, seq_of_token, state_slots, (float*)out, channels, n_taps);
    else if (dtype == PB_BF16)
        launch_pdl(causal_conv_silu_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)in, in_tok, taps, bias, arena,
                                                                         slot_stride, tail_offset, cu_q, seq_of_token, state_slots,
                                                                         (__nv_bfloat16*)out, channels, n_taps);
    else return PB_ERR_BAD_DTYPE;
    return launch_status();
}

// x [N, inner] (the convolution's output), xz [N, xz_tok] (the input projection: convolution inputs in columns
// [0, inner), gates z in [inner, 2 inner)), proj [N, proj_tok] = [r: dt_rank | B: state | C: state], w_dt [inner, dt_rank],
// y [N, inner].  The arena's slot holds [inner, state] and, at tail_offset, [inner, taps - 1].
PB_EXPORT int pb_selective_scan(int dtype, const void* x, const void* xz, long xz_tok, const void* proj, long proj_tok,
                                const void* w_dt, const float* dt_bias, const float* a_log, const float* d_skip, float* arena,
                                long slot_stride, long tail_offset, void* y, const int* cu_q, const int* state_slots, int n_seqs,
                                int inner, int n_state, int dt_rank, int n_taps, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || dt_rank <= 0 || n_taps < 1) return PB_ERR_BAD_SIZE;
    if (n_state > 32 * kStatesPerLane || dt_rank > 32 * kDtPerLane) return PB_ERR_TOO_LARGE;
    if ((size_t)kStage * (2 * n_state + dt_rank + 32) * sizeof(float) > 48 * 1024) return PB_ERR_TOO_LARGE;
    const ScanShape sh{inner, n_state, dt_rank, n_taps, slot_stride, tail_offset, xz_tok, proj_tok};
    if (dtype == PB_F32)
        return dispatch_scan<float>(x, xz, proj, w_dt, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh, stream);
    if (dtype == PB_BF16)
        return dispatch_scan<__nv_bfloat16>(x, xz, proj, w_dt, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh,
                                            stream);
    return PB_ERR_BAD_DTYPE;
}

// 1 when the kernel for portions takes this state size (its staging fits the default shared memory), else 0: the caller
// then uses pb_selective_scan for portions too.
PB_EXPORT int pb_selective_scan_prompt_supported(int n_state) {
    if (n_state <= 0 || n_state > 32 * kStatesPerLane) return 0;
    return (size_t)kStagePrompt * (2 * n_state + 3 * 16) * sizeof(float) <= 48 * 1024 ? 1 : 0;
}

// The same scan with the step sizes' product done beforehand: dt_pre [N, inner] float32 = W_dt r (no bias yet), and
// bc [N, bc_tok] whose rows start with [B: state | C: state].  For steps with prompt portions.
PB_EXPORT int pb_selective_scan_prompt(int dtype, const void* x, const void* xz, long xz_tok, const void* bc, long bc_tok,
                                       const float* dt_pre, const float* dt_bias, const float* a_log, const float* d_skip,
                                       float* arena, long slot_stride, long tail_offset, void* y, const int* cu_q,
                                       const int* state_slots, int n_seqs, int inner, int n_state, int n_taps, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || n_taps < 1) return PB_ERR_BAD_SIZE;
    if (!pb_selective_scan_prompt_supported(n_state)) return PB_ERR_TOO_LARGE;
    const ScanShape sh{inner, n_state, 0, n_taps, slot_stride, tail_offset, xz_tok, 0};
    if (dtype == PB_F32)
        return dispatch_scan_prompt<float>(x, xz, bc, bc_tok, dt_pre, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh,
                                           stream);
    if (dtype == PB_BF16)
        return dispatch_scan_prompt<__nv_bfloat16>(x, xz, bc, bc_tok, dt_pre, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots,
                                                   n_seqs, sh, stream);
    return PB_ERR_BAD_DTYPE;
}

// 1 when the scan that is parallel over tokens takes this state size (its staging of 256 tokens fits the shared memory).
PB_EXPORT int pb_selective_scan_chunked_supported(int n_state) {
    return (n_state > 0 && chunked_smem(n_state) <= 160 * 1024) ? 1 : 0;
}

// pb_selective_scan_prompt's arguments; the recurrence is evaluated 256 tokens at a time with a prefix scan over runs of 8.
PB_EXPORT int pb_selective_scan_chunked(int dtype, const void* x, const void* xz, long xz_tok, const void* bc, long bc_tok,
                                        const float* dt_pre, const float* dt_bias, const float* a_log, const float* d_skip,
                                        float* arena, long slot_stride, long tail_offset, void* y, const int* cu_q,
                                        const int* state_slots, int n_seqs, int inner, int n_state, int n_taps, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (inner <= 0 || n_state <= 0 || n_taps < 1) return PB_ERR_BAD_SIZE;
    if (!pb_selective_scan_chunked_supported(n_state)) return PB_ERR_TOO_LARGE;
    if ((inner + kChunkChannels - 1) / kChunkChannels > 65535) return PB_ERR_TOO_LARGE;
    const ScanShape sh{inner, n_state, 0, n_taps, slot_stride, tail_offset, xz_tok, 0};
    if (dtype == PB_F32)
        return launch_scan_chunked<float>(x, xz, bc, bc_tok, dt_pre, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs, sh, stream);
    if (dtype == PB_BF16)
        return launch_scan_chunked<__nv_bfloat16>(x, xz, bc, bc_tok, dt_pre, dt_bias, a_log, d_skip, arena, y, cu_q, state_slots, n_seqs,
                                                  sh, stream);
    return PB_ERR_BAD_DTYPE;
}
