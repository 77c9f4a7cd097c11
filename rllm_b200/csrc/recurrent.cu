// Layers that carry a fixed-size state per request from token to token: the selective scan
// (Mamba) with its short causal convolution, RWKV-style time mixing with a data-dependent
// decay, retention (linear attention with a fixed decay per head) and the matrix memory with
// exponential gates and a running maximum (mLSTM).  A request's state lives in a slot of the state array (float32), is read at the start of
// the request's tokens in this step and written back at their end; the tokens of a request are
// contiguous in the flat batch (cu_q) and in order.  Everything that enters a recurrence (step
// sizes, decays, their exponentials, gates, unit norms, the state itself) is float32 with accurate
// expf / log1pf; one thread (or a fixed group of lanes) owns a state element for the whole step,
// and sums run in a fixed order, so a request's result does not depend on what else is in the
// batch, on how its tokens were cut into steps, or on the slot it has.
//
// State slot layouts (floats):
//   Mamba:  S [inner][N], then the last taps-1 inputs of the convolution [inner][taps-1] (oldest first)
//   RWKV :  S of every head, DMAX * DMAX floats a head (DMAX: the head size rounded up to 32, 64, 128
//           or 256; rllm_wkv_state_floats) in the order in which the WKV kernel's threads hold it, so
//           that a step reads and writes it in whole lines: value (register, thread) at register *
//           threads + thread; then the previous token's input [width].  Nothing else reads S.
//   retention:  S of every head, DKMAX * dvp floats a head, in the retention kernel's thread order.
//   mlstm:  per head DKMAX * dvp floats in the same order, whose value column dv is the normaliser n, then
//           four floats of which the first is the running maximum m.  Heads beyond the kernel's sizes: S
//           [dk][dv + 1] row-major and the four floats.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ causal convolution + silu
// xz [n, ld] float32 holds the convolution's input in columns [0, inner).  Token t (index i in
// its request's portion) and channel c:
//   out[t, c] = silu(b[c] + sum_j w[c, j] * in(i - (taps-1) + j)),  in(i') = xz row of that token
//   for i' >= 0, else the request's kept inputs (state) -- zeros at the start of a sequence.
// The state itself is advanced by the scan kernel, which runs after every read here.
#define CONV_TOK 1             // tokens per block (more did not pay: 119 us against 116 for 2,048 x 8,192, and decode steps lost)
template <typename TO>
__global__ void conv_silu_kernel(const float* xz, long long ld, const float* __restrict__ w,
                                 const float* __restrict__ b, const float* state, long long slot_stride,
                                 long long conv_off, const int* __restrict__ seq_ids, const int* __restrict__ cu_q,
                                 const int* __restrict__ slots, TO* out, int n, int inner, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    // a block takes CONV_TOK tokens in a row, its threads the channels
    for (int t = blockIdx.x * CONV_TOK; t < min(n, (int)(blockIdx.x + 1) * CONV_TOK); ++t) {
        const int r = seq_ids[t];
        const int i = t - cu_q[r];
        const float* st = state + (size_t)slots[r] * slot_stride + conv_off;
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < inner; c += gridDim.y * blockDim.x) {
            float acc = b ? b[c] : 0.f;
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j;             // how many tokens before this one
                const float v = back <= i ? xz[(size_t)(t - back) * ld + c]
                                          : st[(size_t)c * (taps - 1) + (taps - 1 - (back - i))];
                acc += w[(size_t)c * taps + j] * v;
            }
            out[(size_t)t * inner + c] = from_f<TO>(silu_f(acc));
        }
    }
}

RLLM_API int rllm_conv_silu(const float* xz, long long ld, const float* w, const float* b, const float* state,
                            long long slot_stride, long long conv_off, const int* seq_ids, const int* cu_q,
                            const int* slots, void* out, int out_dt, int n, int inner, int taps,
                            cudaStream_t stream) {
    if (n <= 0) return 0;
    if (taps < 1 || inner <= 0) return (int)cudaErrorInvalidValue;
    const dim3 grid((n + CONV_TOK - 1) / CONV_TOK, (inner + 255) / 256 > 64 ? 64 : (inner + 255) / 256);
    if (out_dt == RLLM_F32)
        return rllm_launch(conv_silu_kernel<float>, grid, dim3(256), 0, stream, xz, ld, w, b, state, slot_stride,
                           conv_off, seq_ids, cu_q, slots, (float*)out, n, inner, taps);
    return rllm_launch(conv_silu_kernel<bf16>, grid, dim3(256), 0, stream, xz, ld, w, b, state, slot_stride, conv_off,
                       seq_ids, cu_q, slots, (bf16*)out, n, inner, taps);
}

// ------------------------------------------------------------------ selective scan
// Per request r, channel c, state index n, over the request's tokens in order:
//   dt = softplus(dtr[t, c] + dt_b[c]);  S[c, n] = exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n]
//   y  = sum_n S[c, n] * C[t, n] + D[c] * x[t, c];      out[t, c] = y * silu(z[t, c])
// x: the convolution's output (activation type), B and C: columns of `low` (float32), z: columns
// [inner, 2 inner) of xz.  SCAN_LANES lanes share a channel (state index n = lane + SCAN_LANES * k);
// their partial sums are added in a fixed butterfly.  A block owns SCAN_CH channels of one request and
// walks its tokens SCAN_TOK at a time: x, the step sizes (softplus done on the way in), silu(z), B and
// C of a chunk lie in shared memory, and the next chunk's values are already on their way from global
// memory (held in registers) while this one is worked through, so the recurrence never waits for a
// load.  At the end the convolution's kept inputs move on by this step's tokens.
// Long portions are also cut along time, as for the WKV kernel below (TimeSegments): a segment
// multiplies the state by exp(A * sum of its step sizes) and adds its end state from a zero start.
// PASS 0: whole requests.  1: the local end state and the sum of the step sizes, no output.  2: from
// the carried start state, with output.
// Segments of the step's requests along time; all null / zero: every request is one item.
struct TimeSegments {
    const int* t0;        // [items] first flat token
    const int* t1;        // [items] one past the last
    const int* req;       // [items] the request's row in the step
    const int* flags;     // [items] bit 0: first segment of its request, bit 1: last
    const int* req_item0; // [requests] a request's first item
    const int* req_items; // [requests] how many it has
    float* carry;         // [items][rows of state per item]: local end states, then true end states
    float* decay;         // [items][...]: what the combine step multiplies the start state by
    int n_items;
};

#define SCAN_LANES 4
#define SCAN_CH 32            // channels per block (128 threads)
#define SCAN_TOK 16           // tokens per chunk
#define SCAN_THREADS (SCAN_LANES * SCAN_CH)

template <typename TA, int NPT, int PASS>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const TA* x, const float* xz, long long ld_xz, const float* low, long long ld_low, int b_off,
                      int c_off, const float* dtr, const float* __restrict__ dt_b, const float* __restrict__ A,
                      const float* __restrict__ Dp, float* state, long long slot_stride, long long conv_off,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, TA* out, int inner, int N,
                      int taps, const TimeSegments seg) {
    constexpr int PRE_X = 3 * SCAN_TOK * SCAN_CH / SCAN_THREADS;      // x, dt, z of a chunk: values per thread
    constexpr int PRE_BC = NPT;                                        // B and C of a chunk (N <= SCAN_LANES * NPT)
    extern __shared__ float sm_scan[];
    float* s_x = sm_scan;                                // [SCAN_TOK][SCAN_CH]
    float* s_dt = s_x + SCAN_TOK * SCAN_CH;
    float* s_z = s_dt + SCAN_TOK * SCAN_CH;              // silu(z)
    float* s_bc = s_z + SCAN_TOK * SCAN_CH;              // [SCAN_TOK][2][N]
    pdl_wait();
    pdl_launch_dependents();
    const int item = blockIdx.y;
    const int r = PASS == 0 ? item : seg.req[item];
    const int t0 = PASS == 0 ? cu_q[r] : seg.t0[item], t1 = PASS == 0 ? cu_q[r + 1] : seg.t1[item];
    const bool first = PASS == 0 || (seg.flags[item] & 1), last = PASS == 0 || (seg.flags[item] & 2);
    if (PASS == 1 && last) return;                       // its end state comes out of pass 2
    const int tid = threadIdx.x, lane = tid % SCAN_LANES, cl = tid / SCAN_LANES;
    const int c_base = blockIdx.x * SCAN_CH;
    const int c_own = c_base + cl;
    const bool live = c_own < inner;
    const int c = live ? c_own : inner - 1;             // lanes beyond the last channel shadow it and write nothing
    float* st = state + (size_t)slots[r] * slot_stride;
    // the start state: the slot; with several segments the combine step's copy of it or the end state of the
    // segment before (the last segment overwrites the slot while the first may not have started)
    const int src = first ? item + (PASS == 0 ? 0 : seg.req_items[r]) - 1 : item - 1;
    const float* from = (first && last) ? st : seg.carry + (size_t)src * inner * N;
    float S[NPT], a[NPT];
    float sum_dt = 0.f;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
        const int n = lane + SCAN_LANES * k;
        const bool on = n < N;
        S[k] = (on && PASS != 1) ? from[(size_t)c * N + n] : 0.f;
        a[k] = on ? A[(size_t)c * N + n] : 0.f;
    }
    const float dd = Dp[c];
    float px[PRE_X], pbc[PRE_BC];
    // element e of the x/dt/z part: which (0 x, 1 dt, 2 z), token, channel of the block
    auto fetch = [&](int tb) {
        const int nt = min(SCAN_TOK, t1 - tb);
#pragma unroll
        for (int i = 0; i < PRE_X; ++i) {
            const int e = tid + i * SCAN_THREADS;
            const int which = e / (SCAN_TOK * SCAN_CH), rem = e % (SCAN_TOK * SCAN_CH);
            const int tt = rem / SCAN_CH, ch = c_base + rem % SCAN_CH;
            float v = 0.f;
            if (tt < nt && ch < inner) {
                const size_t t = tb + tt;
                v = which == 0 ? to_f<TA>(x[t * inner + ch]) : which == 1 ? dtr[t * inner + ch] : xz[t * ld_xz + inner + ch];
            }
            px[i] = v;
        }
#pragma unroll
        for (int i = 0; i < PRE_BC; ++i) {
            const int e = tid + i * SCAN_THREADS;
            const int tt = e / (2 * N), j = e % (2 * N);
            pbc[i] = (tt < nt) ? low[(size_t)(tb + tt) * ld_low + (j < N ? b_off + j : c_off + j - N)] : 0.f;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int i = 0; i < PRE_X; ++i) {
            const int e = tid + i * SCAN_THREADS;
            const int which = e / (SCAN_TOK * SCAN_CH), rem = e % (SCAN_TOK * SCAN_CH);
            const int ch = c_base + rem % SCAN_CH;
            float v = px[i];
            if (which == 1) v = softplus_f(v + (ch < inner ? dt_b[ch] : 0.f));
            else if (which == 2) v = silu_f(v);
            sm_scan[e] = v;
        }
#pragma unroll
        for (int i = 0; i < PRE_BC; ++i) {
            const int e = tid + i * SCAN_THREADS;
            if (e < SCAN_TOK * 2 * N) s_bc[e] = pbc[i];
        }
    };
    if (t0 < t1) {
        fetch(t0);
        stash();
    }
    __syncthreads();
    for (int tb = t0; tb < t1; tb += SCAN_TOK) {
        const int nt = min(SCAN_TOK, t1 - tb);
        const bool more = tb + SCAN_TOK < t1;
        if (more) fetch(tb + SCAN_TOK);
        // One token: only S carries over from the token before, so with the loop unrolled the
        // exponentials, loads and shuffles of neighbouring tokens overlap.
        auto token = [&](int tt) {
            const float xv = s_x[tt * SCAN_CH + cl];
            const float dt = s_dt[tt * SCAN_CH + cl];
            const float dx = dt * xv;
            const float* Bt = s_bc + tt * 2 * N;
            const float* Ct = Bt + N;
            float part = 0.f;
            if (PASS == 1) sum_dt += dt;
#pragma unroll
            for (int k = 0; k < NPT; ++k) {
                const int n = lane + SCAN_LANES * k;
                if (n < N) {
                    S[k] = expf(dt * a[k]) * S[k] + dx * Bt[n];
                    if (PASS != 1) part += S[k] * Ct[n];
                }
            }
            if (PASS == 1) return;
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            if (lane == 0 && live)
                out[(size_t)(tb + tt) * inner + c] = from_f<TA>((part + dd * xv) * s_z[tt * SCAN_CH + cl]);
        };
        if (nt == SCAN_TOK) {
#pragma unroll 4
            for (int tt = 0; tt < SCAN_TOK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        __syncthreads();                                 // everyone is done with this chunk
        if (more) stash();
        __syncthreads();
    }
    if (!live) return;
    if (PASS == 1) {
        float* to = seg.carry + (size_t)item * inner * N;
#pragma unroll
        for (int k = 0; k < NPT; ++k) {
            const int n = lane + SCAN_LANES * k;
            if (n < N) to[(size_t)c * N + n] = S[k];
        }
        if (lane == 0) seg.decay[(size_t)item * inner + c] = sum_dt;
        return;
    }
    if (!last) return;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
        const int n = lane + SCAN_LANES * k;
        if (n < N) st[(size_t)c * N + n] = S[k];
    }
    if (lane == 0 && taps > 1) {
        // kept inputs: the last taps-1 of (old kept inputs ++ this step's inputs), oldest first
        float* cs = st + conv_off + (size_t)c * (taps - 1);
        const int q0 = cu_q[r], q = t1 - q0;             // the request's tokens of this step, all segments
        for (int k = 0; k < taps - 1; ++k) {
            const int idx = q + k;                       // place in the joined sequence
            cs[k] = idx < taps - 1 ? cs[idx] : xz[(size_t)(q0 + idx - (taps - 1)) * ld_xz + c];
        }
    }
}

// Between the passes: a request's segments in order, S_end = exp(A * sum of step sizes) * S_start + local
// end state, in place; the start state is copied to where the last segment's local state would be.
template <int NPT>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_combine_kernel(const float* state, long long slot_stride, const int* __restrict__ slots,
                    const float* __restrict__ A, int inner, int N, const TimeSegments seg) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int n_it = seg.req_items[r], item0 = seg.req_item0[r];
    if (n_it < 2) return;
    const int tid = threadIdx.x, lane = tid % SCAN_LANES;
    const int c = blockIdx.x * SCAN_CH + tid / SCAN_LANES;
    if (c >= inner) return;
    const float* st = state + (size_t)slots[r] * slot_stride;
    float S[NPT], a[NPT];
    float* keep = seg.carry + (size_t)(item0 + n_it - 1) * inner * N;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
        const int n = lane + SCAN_LANES * k;
        S[k] = n < N ? st[(size_t)c * N + n] : 0.f;
        a[k] = n < N ? A[(size_t)c * N + n] : 0.f;
        if (n < N) keep[(size_t)c * N + n] = S[k];
    }
    for (int it = item0; it < item0 + n_it - 1; ++it) {
        float* C = seg.carry + (size_t)it * inner * N;
        const float sum_dt = seg.decay[(size_t)it * inner + c];
#pragma unroll
        for (int k = 0; k < NPT; ++k) {
            const int n = lane + SCAN_LANES * k;
            if (n < N) {
                S[k] = expf(sum_dt * a[k]) * S[k] + C[(size_t)c * N + n];
                C[(size_t)c * N + n] = S[k];
            }
        }
    }
}

template <typename TA, int NPT>
static int launch_scan(int n_requests, size_t smem, cudaStream_t stream, const void* x, const float* xz, long long ld_xz,
                       const float* low, long long ld_low, int b_off, int c_off, const float* dtr, const float* dt_b,
                       const float* A, const float* Dp, float* state, long long slot_stride, long long conv_off,
                       const int* cu_q, const int* slots, void* out, int inner, int N, int taps, const TimeSegments& seg) {
    const int cols = (inner + SCAN_CH - 1) / SCAN_CH;
#define SCAN_ARGS (const TA*)x, xz, ld_xz, low, ld_low, b_off, c_off, dtr, dt_b, A, Dp, state, slot_stride, conv_off, cu_q, \
                  slots, (TA*)out, inner, N, taps, seg
    if (seg.n_items <= 0)
        return rllm_launch(selective_scan_kernel<TA, NPT, 0>, dim3(cols, n_requests), dim3(SCAN_THREADS), smem, stream, SCAN_ARGS);
    int st = rllm_launch(selective_scan_kernel<TA, NPT, 1>, dim3(cols, seg.n_items), dim3(SCAN_THREADS), smem, stream, SCAN_ARGS);
    if (st) return st;
    st = rllm_launch(scan_combine_kernel<NPT>, dim3(cols, n_requests), dim3(SCAN_THREADS), 0, stream, (const float*)state,
                     slot_stride, slots, A, inner, N, seg);
    if (st) return st;
    return rllm_launch(selective_scan_kernel<TA, NPT, 2>, dim3(cols, seg.n_items), dim3(SCAN_THREADS), smem, stream, SCAN_ARGS);
#undef SCAN_ARGS
}

// seg_* / carry / decay: the cut along time (TimeSegments; n_items 0: none).  carry needs n_items * inner * N
// floats, decay n_items * inner.
RLLM_API int rllm_selective_scan(const void* x, int act_dt, const float* xz, long long ld_xz, const float* low,
                                 long long ld_low, int b_off, int c_off, const float* dtr, const float* dt_b,
                                 const float* A, const float* Dp, float* state, long long slot_stride,
                                 long long conv_off, const int* cu_q, const int* slots, void* out, int n_requests,
                                 int inner, int N, int taps, const int* seg_t0, const int* seg_t1, const int* seg_req,
                                 const int* seg_flags, const int* req_item0, const int* req_items, int n_items,
                                 float* carry, float* decay, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (N <= 0 || N > SCAN_LANES * 64 || inner <= 0 || taps < 1) return (int)cudaErrorInvalidValue;
    TimeSegments seg = {seg_t0, seg_t1, seg_req, seg_flags, req_item0, req_items, carry, decay, n_items};
    if (n_items > 0 && (!seg_t0 || !seg_t1 || !seg_req || !seg_flags || !req_item0 || !req_items || !carry || !decay))
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(3 * SCAN_TOK * SCAN_CH + SCAN_TOK * 2 * N) * sizeof(float);
#define LAUNCH(TA, NPT)                                                                                          \
    return launch_scan<TA, NPT>(n_requests, smem, stream, x, xz, ld_xz, low, ld_low, b_off, c_off, dtr, dt_b, A, Dp, \
                                state, slot_stride, conv_off, cu_q, slots, out, inner, N, taps, seg)
#define BY_N(TA)                                                                                                 \
    do {                                                                                                         \
        if (N <= SCAN_LANES * 4) { LAUNCH(TA, 4); }                                                              \
        if (N <= SCAN_LANES * 8) { LAUNCH(TA, 8); }                                                              \
        if (N <= SCAN_LANES * 16) { LAUNCH(TA, 16); }                                                            \
        if (N <= SCAN_LANES * 32) { LAUNCH(TA, 32); }                                                            \
        LAUNCH(TA, 64);                                                                                          \
    } while (0)
    if (act_dt == RLLM_F32) BY_N(float);
    BY_N(bf16);
#undef BY_N
#undef LAUNCH
}

// ------------------------------------------------------------------ token shift
// out[s][t, c] = h[t, c] + (prev(t)[c] - h[t, c]) * mu[s][c] for s < n_streams; prev(t) is the row
// before t of the same request, or the request's kept row (state) for the first token of its
// portion -- zeros at the start of a sequence.  The kept row is advanced by the WKV kernel.
template <typename TA>
__global__ void token_shift_kernel(const TA* h, const float* __restrict__ mu, const float* state,
                                   long long slot_stride, long long prev_off, const int* __restrict__ seq_ids,
                                   const int* __restrict__ cu_q, const int* __restrict__ slots, TA* out, int n, int d,
                                   int n_streams) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int r = seq_ids[t];
    const bool first = t == cu_q[r];
    const float* pv = state + (size_t)slots[r] * slot_stride + prev_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < d; c += gridDim.y * blockDim.x) {
        const float cur = to_f<TA>(h[(size_t)t * d + c]);
        const float prev = first ? pv[c] : to_f<TA>(h[(size_t)(t - 1) * d + c]);
        for (int s = 0; s < n_streams; ++s)
            out[((size_t)s * n + t) * d + c] = from_f<TA>(cur + (prev - cur) * mu[(size_t)s * d + c]);
    }
}

RLLM_API int rllm_token_shift(const void* h, int act_dt, const float* mu, const float* state, long long slot_stride,
                              long long prev_off, const int* seq_ids, const int* cu_q, const int* slots, void* out,
                              int n, int d, int n_streams, cudaStream_t stream) {
    if (n <= 0) return 0;
    // few tokens (a decode step): the row is spread over several blocks; many: a block per row
    // (2,048 x 4,096: 62 us against 81 with sixteen blocks a row)
    const dim3 grid(n, n >= 256 ? 1 : (d + 255) / 256 > 32 ? 32 : (d + 255) / 256);
    if (act_dt == RLLM_F32)
        return rllm_launch(token_shift_kernel<float>, grid, dim3(256), 0, stream, (const float*)h, mu, state,
                           slot_stride, prev_off, seq_ids, cu_q, slots, (float*)out, n, d, n_streams);
    return rllm_launch(token_shift_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)h, mu, state,
                       slot_stride, prev_off, seq_ids, cu_q, slots, (bf16*)out, n, d, n_streams);
}

// ------------------------------------------------------------------ WKV with data-dependent decay
// One block per (request, head).  Per token, with r, k, v the head's rows of the projections,
// w = exp(-exp(wraw + w0)) the decay per key channel and u the bonus of the current token:
//   o[j] = sum_i r[i] * (S[i][j] + u[i] * k[i] * v[j]);     S[i][j] = w[i] * S[i][j] + k[i] * v[j]
// then o is divided by its root mean square over the head (eps inside the root), multiplied by the
// norm weight and by silu(gate), and stored in the activation type.  The bonus term is the same
// number for every value channel, o[j] = sum_i r[i] S[i][j] + (sum_i r[i] u[i] k[i]) * v[j], and is
// worked out once per token.
// A thread owns an eighth of the key channels (DMAX / 8) of two neighbouring value channels of the
// state, in registers: r, k and w are read once for both columns (the kernel is bound by those
// reads), and the WKV_PARTS lanes that share a pair of columns add their partial sums in a fixed
// butterfly.  Tokens are taken WKV_TOK at a time: r, k, the decay (exponentials done on the way in),
// v and the gate of a chunk lie in shared memory (rows padded with zeros to DMAX, read four at a
// time), the next chunk's values are already on their way from global memory (held in registers)
// while this one is worked through, and the chunk's outputs are normalised by the warps in turn.
// The kept previous row moves on at the end.
//
// Long portions are also cut along time (TimeSegments): the decay is diagonal, so a segment's effect on
// the state is  S_end = diag(prod of its decays) S_start + (its end state from a zero start).  Pass 1
// works out the second term and the product for every segment but a request's last, all segments side
// by side; a small kernel then walks each request's segments and turns the local end states into true
// ones; pass 2 runs every segment from its true start state and writes the outputs (the last one also
// the request's state).  Twice the arithmetic, as many blocks as segments x heads.  The sums inside a
// segment run in the same order as without the cut; across the cut they are associated differently,
// which moves results by rounding only.
#define WKV_TOK 16
#define WKV_PARTS 8
#define WKV_COLS 2

// PASS 0: whole requests.  1: end state from a zero start and the product of the decays, no output.
// 2: from the carried start state, with output.
template <typename TA, int DMAX, int PASS>
__global__ void __launch_bounds__(WKV_PARTS * DMAX / WKV_COLS, DMAX <= 64 ? 4 : 1)
wkv_kernel(const float* rp, const float* kp, const float* vp, const float* wraw, const float* gp, long long ld,
           const float* __restrict__ w0, const float* __restrict__ u, const float* __restrict__ norm_w, float eps,
           float* state, long long slot_stride, long long prev_off, const TA* h, int width,
           const int* __restrict__ cu_q, const int* __restrict__ slots, TA* out, int H, int D,
           const TimeSegments seg) {
    constexpr int IPT = DMAX / WKV_PARTS;               // key channels per thread
    constexpr int NT = WKV_PARTS * DMAX / WKV_COLS;     // threads
    constexpr int TD = WKV_TOK * DMAX;
    constexpr int PRE = 5 * TD / NT;                    // values a thread brings in per chunk
    extern __shared__ __align__(16) float sm_wkv[];      // r, k, w, v, gate: [5][WKV_TOK][DMAX]; o: [WKV_TOK][DMAX]; u: [DMAX]; bonus: [WKV_TOK]
    float* s_r = sm_wkv;
    float* s_k = s_r + TD;
    float* s_w = s_k + TD;
    float* s_v = s_w + TD;
    float* s_g = s_v + TD;
    float* s_o = s_g + TD;
    float* s_u = s_o + TD;
    float* s_c = s_u + DMAX;
    const int tid = threadIdx.x, j0 = WKV_COLS * (tid / WKV_PARTS), part = tid % WKV_PARTS;
    const int head = blockIdx.x, item = blockIdx.y;
    const size_t col = (size_t)head * D;
    for (int i = tid; i < DMAX; i += NT) s_u[i] = i < D ? u[col + i] : 0.f;
    pdl_wait();
    pdl_launch_dependents();
    const int r = PASS == 0 ? item : seg.req[item];
    const int t0 = PASS == 0 ? cu_q[r] : seg.t0[item], t1 = PASS == 0 ? cu_q[r + 1] : seg.t1[item];
    const bool first = PASS == 0 || (seg.flags[item] & 1), last = PASS == 0 || (seg.flags[item] & 2);
    if (PASS == 1 && last) return;                       // its end state comes out of pass 2
    float* st = state + (size_t)slots[r] * slot_stride;
    float* Sg = st + (size_t)head * DMAX * DMAX;
    const int i0 = part * IPT;
    // key channels i0 .. i0 + IPT of the value channels j0 and j0 + 1; what lies beyond D stays zero
    float S0[IPT], S1[IPT], cw[PASS == 1 ? IPT : 1];
    {
        // A request's start state: in its slot; with several segments the combine step has put a copy
        // where the last segment's local state would be, because the last segment overwrites the slot
        // while the first may not have started.
        const int src = first ? item + seg.req_items[r] - 1 : item - 1;
        const float* from = (first && last) ? Sg : seg.carry + ((size_t)src * H + head) * DMAX * DMAX;
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            S0[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii) * NT + tid];
            S1[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii + 1) * NT + tid];
            if (PASS == 1) cw[ii] = 1.f;
        }
    }
    float pre[PRE];
    auto fetch = [&](int tb) {
        const int nt = min(WKV_TOK, t1 - tb);
#pragma unroll
        for (int x = 0; x < PRE; ++x) {
            const int e = tid + x * NT;
            const int arr = e / TD, rem = e % TD, tt = rem / DMAX, cc = rem % DMAX;
            const float* src = arr == 0 ? rp : arr == 1 ? kp : arr == 2 ? wraw : arr == 3 ? vp : gp;
            pre[x] = (tt < nt && cc < D) ? src[(size_t)(tb + tt) * ld + col + cc] : 0.f;
        }
    };
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int n_warps = NT / 32;
    // the chunk's values into shared memory, then the bonus sums of its tokens, a warp per token
    auto stash = [&]() {
#pragma unroll
        for (int x = 0; x < PRE; ++x) {
            const int e = tid + x * NT;
            const int arr = e / TD, cc = e % DMAX;
            float v = pre[x];
            if (arr == 2) v = cc < D ? expf(-expf(v + w0[col + cc])) : 0.f;
            sm_wkv[e] = v;
        }
        __syncthreads();
        for (int tt = warp; tt < WKV_TOK; tt += n_warps) {
            float c = 0.f;
            for (int i = lane; i < D; i += 32) c += s_r[tt * DMAX + i] * s_u[i] * s_k[tt * DMAX + i];
            c = warp_sum(c);
            if (lane == 0) s_c[tt] = c;
        }
    };
    if (t0 < t1) fetch(t0);
    __syncthreads();                                     // s_u is there
    if (t0 < t1) stash();
    __syncthreads();
    for (int tb = t0; tb < t1; tb += WKV_TOK) {
        const int nt = min(WKV_TOK, t1 - tb);
        const bool more = tb + WKV_TOK < t1;
        if (more) fetch(tb + WKV_TOK);
        // One token: only S carries over from the token before, so with the loop unrolled the loads and
        // products of neighbouring tokens overlap.
        auto token = [&](int tt) {
            const float2 vj = *reinterpret_cast<const float2*>(s_v + tt * DMAX + j0);
            const float4* r4 = reinterpret_cast<const float4*>(s_r + tt * DMAX + i0);
            const float4* k4 = reinterpret_cast<const float4*>(s_k + tt * DMAX + i0);
            const float4* w4 = reinterpret_cast<const float4*>(s_w + tt * DMAX + i0);
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int q = 0; q < IPT / 4; ++q) {
                const float4 rr = r4[q], kk = k4[q], ww = w4[q];
#define WKV_STEP(R, K, W, I, A, B)                                   \
                if (PASS != 1) { A += R * S0[I]; B += R * S1[I]; }   \
                else cw[I] *= W;                                     \
                S0[I] = W * S0[I] + K * vj.x; S1[I] = W * S1[I] + K * vj.y;
                WKV_STEP(rr.x, kk.x, ww.x, 4 * q, a0, b0)
                WKV_STEP(rr.y, kk.y, ww.y, 4 * q + 1, a1, b1)
                WKV_STEP(rr.z, kk.z, ww.z, 4 * q + 2, a0, b0)
                WKV_STEP(rr.w, kk.w, ww.w, 4 * q + 3, a1, b1)
#undef WKV_STEP
            }
            if (PASS == 1) return;
            float oa = a0 + a1, ob = b0 + b1;
#pragma unroll
            for (int m = 1; m < WKV_PARTS; m <<= 1) {
                oa += __shfl_xor_sync(0xffffffffu, oa, m);
                ob += __shfl_xor_sync(0xffffffffu, ob, m);
            }
            if (part == 0) {
                const float c = s_c[tt];
                *reinterpret_cast<float2*>(s_o + tt * DMAX + j0) = make_float2(oa + c * vj.x, ob + c * vj.y);
            }
        };
        if (nt == WKV_TOK) {
#pragma unroll 2
            for (int tt = 0; tt < WKV_TOK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        __syncthreads();
        for (int tt = warp; PASS != 1 && tt < nt; tt += n_warps) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) ss += s_o[tt * DMAX + i] * s_o[tt * DMAX + i];
            const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
            for (int i = lane; i < D; i += 32)
                out[(size_t)(tb + tt) * H * D + col + i] =
                    from_f<TA>(s_o[tt * DMAX + i] * rs * norm_w[col + i] * silu_f(s_g[tt * DMAX + i]));
        }
        __syncthreads();                                 // everyone is done with this chunk
        if (more) stash();
        __syncthreads();
    }
    if (PASS == 1) {
        float* to = seg.carry + ((size_t)item * H + head) * DMAX * DMAX;
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            to[(size_t)(2 * ii) * NT + tid] = S0[ii];
            to[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
            if (tid < WKV_PARTS) seg.decay[((size_t)item * H + head) * DMAX + i0 + ii] = cw[ii];
        }
        return;
    }
    if (!last) return;
#pragma unroll
    for (int ii = 0; ii < IPT; ++ii) {
        Sg[(size_t)(2 * ii) * NT + tid] = S0[ii];
        Sg[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
    }
    if (head == 0 && t1 > t0) {
        float* pv = st + prev_off;
        for (int c = tid; c < width; c += NT) pv[c] = to_f<TA>(h[(size_t)(t1 - 1) * width + c]);
    }
}

// Between the passes: a request's segments in order, S_end = decay * S_start + local end state, in place.
template <int DMAX>
__global__ void __launch_bounds__(WKV_PARTS * DMAX / WKV_COLS)
wkv_combine_kernel(const float* state, long long slot_stride, const int* __restrict__ slots, int H, const TimeSegments seg) {
    constexpr int IPT = DMAX / WKV_PARTS;
    constexpr int NT = WKV_PARTS * DMAX / WKV_COLS;
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, head = blockIdx.x, r = blockIdx.y;
    const int n = seg.req_items[r], item0 = seg.req_item0[r];
    if (n < 2) return;
    const float* Sg = state + (size_t)slots[r] * slot_stride + (size_t)head * DMAX * DMAX;
    const int i0 = (tid % WKV_PARTS) * IPT;
    float S0[IPT], S1[IPT];
#pragma unroll
    for (int ii = 0; ii < IPT; ++ii) {
        S0[ii] = Sg[(size_t)(2 * ii) * NT + tid];
        S1[ii] = Sg[(size_t)(2 * ii + 1) * NT + tid];
    }
    {
        float* keep = seg.carry + ((size_t)(item0 + n - 1) * H + head) * DMAX * DMAX;    // the start state, for pass 2
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            keep[(size_t)(2 * ii) * NT + tid] = S0[ii];
            keep[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
        }
    }
    for (int it = item0; it < item0 + n - 1; ++it) {
        float* C = seg.carry + ((size_t)it * H + head) * DMAX * DMAX;
        const float* dec = seg.decay + ((size_t)it * H + head) * DMAX + i0;
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            const float w = dec[ii];
            S0[ii] = w * S0[ii] + C[(size_t)(2 * ii) * NT + tid];
            S1[ii] = w * S1[ii] + C[(size_t)(2 * ii + 1) * NT + tid];
            C[(size_t)(2 * ii) * NT + tid] = S0[ii];
            C[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
        }
    }
}

template <typename TA, int DMAX, int PASS>
static int launch_wkv_pass(dim3 grid, size_t smem, cudaStream_t stream, const float* rp, const float* kp,
                           const float* vp, const float* wraw, const float* gp, long long ld, const float* w0,
                           const float* u, const float* norm_w, float eps, float* state, long long slot_stride,
                           long long prev_off, const void* h, int width, const int* cu_q, const int* slots, void* out,
                           int H, int D, const TimeSegments& seg) {
    if (smem > 48 * 1024) {
        static bool raised = false;                      // once per instantiation: more dynamic shared memory than the default
        if (!raised) {
            cudaError_t e = cudaFuncSetAttribute(wkv_kernel<TA, DMAX, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = true;
        }
    }
    return rllm_launch(wkv_kernel<TA, DMAX, PASS>, grid, dim3(WKV_PARTS * DMAX / WKV_COLS), smem, stream, rp, kp, vp, wraw,
                       gp, ld, w0, u, norm_w, eps, state, slot_stride, prev_off, (const TA*)h, width, cu_q, slots, (TA*)out,
                       H, D, seg);
}

template <typename TA, int DMAX>
static int launch_wkv(int n_requests, size_t smem, cudaStream_t stream, const float* rp, const float* kp, const float* vp,
                      const float* wraw, const float* gp, long long ld, const float* w0, const float* u,
                      const float* norm_w, float eps, float* state, long long slot_stride, long long prev_off,
                      const void* h, int width, const int* cu_q, const int* slots, void* out, int H, int D,
                      const TimeSegments& seg) {
#define WKV_ARGS rp, kp, vp, wraw, gp, ld, w0, u, norm_w, eps, state, slot_stride, prev_off, h, width, cu_q, slots, out, H, D, seg
    if (seg.n_items <= 0)
        return launch_wkv_pass<TA, DMAX, 0>(dim3(H, n_requests), smem, stream, WKV_ARGS);
    int st = launch_wkv_pass<TA, DMAX, 1>(dim3(H, seg.n_items), smem, stream, WKV_ARGS);
    if (st) return st;
    st = rllm_launch(wkv_combine_kernel<DMAX>, dim3(H, n_requests), dim3(WKV_PARTS * DMAX / WKV_COLS), 0, stream,
                     (const float*)state, slot_stride, slots, H, seg);
    if (st) return st;
    return launch_wkv_pass<TA, DMAX, 2>(dim3(H, seg.n_items), smem, stream, WKV_ARGS);
#undef WKV_ARGS
}

// seg_* / carry / decay: the cut along time (TimeSegments; n_items 0: none).  carry needs n_items * H * DMAX * DMAX
// floats, decay n_items * H * DMAX (DMAX as in rllm_wkv_state_floats).
RLLM_API int rllm_wkv(const float* rp, const float* kp, const float* vp, const float* wraw, const float* gp,
                      long long ld, const float* w0, const float* u, const float* norm_w, float eps, float* state,
                      long long slot_stride, long long prev_off, const void* h, int act_dt, int width,
                      const int* cu_q, const int* slots, void* out, int n_requests, int H, int D,
                      const int* seg_t0, const int* seg_t1, const int* seg_req, const int* seg_flags,
                      const int* req_item0, const int* req_items, int n_items, float* carry, float* decay,
                      cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (D <= 0 || D > 256 || H <= 0) return (int)cudaErrorInvalidValue;
    const int dmax = D <= 32 ? 32 : D <= 64 ? 64 : D <= 128 ? 128 : 256;
    if (prev_off < (long long)H * dmax * dmax) return (int)cudaErrorInvalidValue;
    TimeSegments seg = {seg_t0, seg_t1, seg_req, seg_flags, req_item0, req_items, carry, decay, n_items};
    if (n_items > 0 && (!seg_t0 || !seg_t1 || !seg_req || !seg_flags || !req_item0 || !req_items || !carry || !decay))
        return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)(6 * WKV_TOK + 1) * dmax + WKV_TOK) * sizeof(float);
#define LAUNCH(TA, DMAX)                                                                                        \
    return launch_wkv<TA, DMAX>(n_requests, smem, stream, rp, kp, vp, wraw, gp, ld, w0, u, norm_w, eps, state,  \
                                slot_stride, prev_off, h, width, cu_q, slots, out, H, D, seg)
#define BY_D(TA)                                                                                               \
    do {                                                                                                       \
        if (dmax == 32) { LAUNCH(TA, 32); }                                                                    \
        if (dmax == 64) { LAUNCH(TA, 64); }                                                                    \
        if (dmax == 128) { LAUNCH(TA, 128); }                                                                  \
        LAUNCH(TA, 256);                                                                                       \
    } while (0)
    if (act_dt == RLLM_F32) BY_D(float);
    BY_D(bf16);
#undef BY_D
#undef LAUNCH
}

// Floats of a request's WKV state for H heads of size D (what precedes the kept previous row in the slot).
RLLM_API long long rllm_wkv_state_floats(int H, int D) {
    const int dmax = D <= 32 ? 32 : D <= 64 ? 64 : D <= 128 ? 128 : 256;
    return (long long)H * dmax * dmax;
}

// ------------------------------------------------------------------ retention: linear attention with a fixed decay per head
// One block per (request or segment, head).  Per token, with q, k the head's rows of the projections
// (dk entries) after their rotation, k also multiplied by key_scale, v the head's values (dv entries)
// and c the head's decay:
//   S[i][j] = c * S[i][j] + k[i] * v[j];     o[j] = sum_i q[i] * S[i][j]        (S after the update)
// then o is divided by its root mean square over the head (eps inside the root), multiplied by
// silu(gate) and stored in the activation type.  The rotation turns the first `rot` entries of q and
// k by the token's angles (pairs (i, i + rot/2), or (2i, 2i + 1) when `pairs`) and is done here, on the
// chunk in shared memory, so q and k come in as projected.
// A thread owns an eighth of the key channels (DKMAX / 8, in runs of four that interleave with the
// other seven lanes' so that their float4 reads of q and k fall side by side) of two neighbouring value
// channels of the state, in registers; the RET_PARTS lanes that share a pair of columns add their
// partial sums in a fixed butterfly.  The block has 8 * ceil(dv / 2) threads (rounded up to whole
// warps).  Tokens are taken RET_TOK at a time through two buffers of shared memory filled by cp.async:
// the next chunk is on its way while this one is worked through.  The state of a head lies in the slot
// in the threads' own order, DKMAX * dvp floats a head (dvp: dv rounded up to a multiple of 8;
// rllm_retention_state_floats).
// Long portions are cut along time as for the WKV kernel (TimeSegments): S_end = c^len * S_start +
// (end state from a zero start); the power is worked out in double precision.
#define RET_TOK 16
#define RET_PARTS 8

__device__ __forceinline__ void ret_cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

template <typename TA, int DKMAX, int PASS, int MAXT>
__global__ void __launch_bounds__(MAXT)
retention_kernel(const float* qp, const float* kp, const float* vp, const float* gp, long long ld,
                 const float2* cs_table, int rot, int pairs, float key_scale, const float* __restrict__ decay, float eps,
                 float* state, long long slot_stride, const int* __restrict__ cu_q, const int* __restrict__ slots,
                 TA* out, int H, int dk, int dv, int gate, const TimeSegments seg) {
    constexpr int IPT = DKMAX / RET_PARTS;
    extern __shared__ __align__(16) float sm_ret[];
    const int NT = blockDim.x, dvp = NT / RET_PARTS * 2;
    const int stage = RET_TOK * (2 * DKMAX + 2 * dvp);
    float* s_o = sm_ret + 2 * stage;                      // [RET_TOK][dvp]
    const int tid = threadIdx.x, j0 = 2 * (tid / RET_PARTS), part = tid % RET_PARTS;
    const int head = blockIdx.x, item = blockIdx.y;
    const float c = decay[head];
    pdl_wait();
    pdl_launch_dependents();
    const int r = PASS == 0 ? item : seg.req[item];
    const int t0 = PASS == 0 ? cu_q[r] : seg.t0[item], t1 = PASS == 0 ? cu_q[r + 1] : seg.t1[item];
    const bool first = PASS == 0 || (seg.flags[item] & 1), last = PASS == 0 || (seg.flags[item] & 2);
    if (PASS == 1 && last) return;                        // its end state comes out of pass 2
    const size_t per_head = (size_t)DKMAX * dvp;
    float* Sg = state + (size_t)slots[r] * slot_stride + (size_t)head * per_head;
    float S0[IPT], S1[IPT];
    {
        const int src = first ? item + seg.req_items[r] - 1 : item - 1;
        const float* from = (first && last) ? Sg : seg.carry + ((size_t)src * H + head) * per_head;
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            S0[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii) * NT + tid];
            S1[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii + 1) * NT + tid];
        }
    }
    const size_t qcol = (size_t)head * dk, vcol = (size_t)head * dv;
    // a chunk's q, k (rows of DKMAX, zeros beyond dk), v and gate (rows of dvp) into a buffer
    auto issue = [&](int tb, int buf) {
        float* base = sm_ret + buf * stage;
        const int nt = min(RET_TOK, t1 - tb);
        for (int e = tid; e < 2 * RET_TOK * DKMAX; e += NT) {
            const int arr = e / (RET_TOK * DKMAX), rem = e % (RET_TOK * DKMAX), tt = rem / DKMAX, cc = rem % DKMAX;
            if (tt < nt && cc < dk) ret_cp_async4(base + e, (arr ? kp : qp) + (size_t)(tb + tt) * ld + qcol + cc);
            else base[e] = 0.f;
        }
        float* vb = base + 2 * RET_TOK * DKMAX;
        for (int e = tid; e < 2 * RET_TOK * dvp; e += NT) {
            const int arr = e / (RET_TOK * dvp), rem = e % (RET_TOK * dvp), tt = rem / dvp, cc = rem % dvp;
            if (tt < nt && cc < dv && (arr == 0 || gp)) ret_cp_async4(vb + e, (arr ? gp : vp) + (size_t)(tb + tt) * ld + vcol + cc);
            else vb[e] = 0.f;
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    const int warp = tid >> 5, lane = tid & 31, n_warps = NT >> 5;
    const int half = rot >> 1;
    if (t0 < t1) issue(t0, 0);
    int buf = 0;
    for (int tb = t0; tb < t1; tb += RET_TOK, buf ^= 1) {
        const int nt = min(RET_TOK, t1 - tb);
        const bool more = tb + RET_TOK < t1;
        if (more) {
            issue(tb + RET_TOK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        float* s_q = sm_ret + buf * stage;
        float* s_k = s_q + RET_TOK * DKMAX;
        float* s_v = s_k + RET_TOK * DKMAX;
        float* s_g = s_v + RET_TOK * dvp;
        // the rotation of q and k, and the keys' scale
        for (int e = tid; e < 2 * nt * half; e += NT) {
            const int arr = e / (nt * half), rem = e % (nt * half), tt = rem / half, i = rem % half;
            const float2 a = cs_table[(size_t)(tb + tt) * half + i];
            float* row = (arr ? s_k : s_q) + tt * DKMAX;
            const int iu = pairs ? 2 * i : i, iv = pairs ? 2 * i + 1 : i + half;
            const float u = row[iu], x = row[iv];
            row[iu] = u * a.x - x * a.y;
            row[iv] = x * a.x + u * a.y;
        }
        __syncthreads();
        if (key_scale != 1.f)
            for (int e = tid; e < nt * DKMAX; e += NT) s_k[e] *= key_scale;
        __syncthreads();
        auto token = [&](int tt) {
            const float2 vj = *reinterpret_cast<const float2*>(s_v + tt * dvp + j0);
            const float4* q4 = reinterpret_cast<const float4*>(s_q + tt * DKMAX);
            const float4* k4 = reinterpret_cast<const float4*>(s_k + tt * DKMAX);
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int q = 0; q < IPT / 4; ++q) {
                const float4 qq = q4[part + RET_PARTS * q], kk = k4[part + RET_PARTS * q];
#define RET_STEP(Q, K, I, A, B)                                                  \
                S0[I] = c * S0[I] + K * vj.x; S1[I] = c * S1[I] + K * vj.y;      \
                if (PASS != 1) { A += Q * S0[I]; B += Q * S1[I]; }
                RET_STEP(qq.x, kk.x, 4 * q, a0, b0)
                RET_STEP(qq.y, kk.y, 4 * q + 1, a1, b1)
                RET_STEP(qq.z, kk.z, 4 * q + 2, a0, b0)
                RET_STEP(qq.w, kk.w, 4 * q + 3, a1, b1)
#undef RET_STEP
            }
            if (PASS == 1) return;
            float oa = a0 + a1, ob = b0 + b1;
#pragma unroll
            for (int m = 1; m < RET_PARTS; m <<= 1) {
                oa += __shfl_xor_sync(0xffffffffu, oa, m);
                ob += __shfl_xor_sync(0xffffffffu, ob, m);
            }
            if (part == 0) *reinterpret_cast<float2*>(s_o + tt * dvp + j0) = make_float2(oa, ob);
        };
        if (nt == RET_TOK) {
#pragma unroll 2
            for (int tt = 0; tt < RET_TOK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        __syncthreads();
        for (int tt = warp; PASS != 1 && tt < nt; tt += n_warps) {
            float ss = 0.f;
            for (int i = lane; i < dv; i += 32) ss += s_o[tt * dvp + i] * s_o[tt * dvp + i];
            const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
            for (int i = lane; i < dv; i += 32) {
                float v = s_o[tt * dvp + i] * rs;
                if (gate == 1) v *= silu_f(s_g[tt * dvp + i]);
                else if (gate == 2) v *= 1.0f / (1.0f + expf(-s_g[tt * dvp + i]));
                out[(size_t)(tb + tt) * H * dv + vcol + i] = from_f<TA>(v);
            }
        }
        __syncthreads();                                  // everyone is done with this buffer and with s_o
    }
    float* to = PASS == 1 ? seg.carry + ((size_t)item * H + head) * per_head : Sg;
    if (PASS != 1 && !last) return;
#pragma unroll
    for (int ii = 0; ii < IPT; ++ii) {
        to[(size_t)(2 * ii) * NT + tid] = S0[ii];
        to[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
    }
}

// Between the passes: a request's segments in order, S_end = c^len * S_start + local end state, in place.
// Every entry of the state goes its own way, so the entries of a head are spread over blockIdx.z: a
// thread carries one entry through the request's segments.  per_head = DKMAX * dvp floats.
#define RET_COMBINE_THREADS 256
__global__ void __launch_bounds__(RET_COMBINE_THREADS)
retention_combine_kernel(const float* state, long long slot_stride, const int* __restrict__ slots,
                         const float* __restrict__ decay, int H, int per_head, const TimeSegments seg) {
    pdl_wait();
    pdl_launch_dependents();
    const int head = blockIdx.x, r = blockIdx.y;
    const int i = blockIdx.z * RET_COMBINE_THREADS + threadIdx.x;
    const int n = seg.req_items[r], item0 = seg.req_item0[r];
    if (n < 2 || i >= per_head) return;
    float S = state[(size_t)slots[r] * slot_stride + (size_t)head * per_head + i];
    seg.carry[((size_t)(item0 + n - 1) * H + head) * per_head + i] = S;           // the start state, for pass 2
    const double c = (double)decay[head];
    float w = 0.f;
    int len = -1;
    for (int it = item0; it < item0 + n - 1; ++it) {
        float* C = seg.carry + ((size_t)it * H + head) * per_head + i;
        if (seg.t1[it] - seg.t0[it] != len) {
            len = seg.t1[it] - seg.t0[it];
            w = (float)pow(c, (double)len);
        }
        S = w * S + *C;
        *C = S;
    }
}

static inline int ret_dkmax(int dk) { return dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 128 ? 128 : 256; }
static inline int ret_threads(int dv) { return ((dv + 1) / 2 * RET_PARTS + 31) / 32 * 32; }

template <typename TA, int DKMAX, int PASS, int MAXT>
static int launch_retention_pass(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* qp,
                                 const float* kp, const float* vp, const float* gp, long long ld, const void* cs_table,
                                 int rot, int pairs, float key_scale, const float* decay, float eps, float* state,
                                 long long slot_stride, const int* cu_q, const int* slots, void* out, int H, int dk, int dv,
                                 int gate, const TimeSegments& seg) {
    if (smem > 48 * 1024) {
        static size_t raised = 0;                         // per instantiation: more dynamic shared memory than the default
        if (smem > raised) {
            cudaError_t e = cudaFuncSetAttribute(retention_kernel<TA, DKMAX, PASS, MAXT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = smem;
        }
    }
    return rllm_launch(retention_kernel<TA, DKMAX, PASS, MAXT>, grid, dim3(threads), smem, stream, qp, kp, vp, gp, ld,
                       (const float2*)cs_table, rot, pairs, key_scale, decay, eps, state, slot_stride, cu_q, slots,
                       (TA*)out, H, dk, dv, gate, seg);
}

template <typename TA, int DKMAX, int MAXT>
static int launch_retention(int n_requests, int threads, size_t smem, cudaStream_t stream, const float* qp, const float* kp,
                            const float* vp, const float* gp, long long ld, const void* cs_table, int rot, int pairs,
                            float key_scale, const float* decay, float eps, float* state, long long slot_stride,
                            const int* cu_q, const int* slots, void* out, int H, int dk, int dv, int gate,
                            const TimeSegments& seg) {
#define RET_ARGS qp, kp, vp, gp, ld, cs_table, rot, pairs, key_scale, decay, eps, state, slot_stride, cu_q, slots, out, H, dk, dv, gate, seg
    if (seg.n_items <= 0)
        return launch_retention_pass<TA, DKMAX, 0, MAXT>(dim3(H, n_requests), threads, smem, stream, RET_ARGS);
    int st = launch_retention_pass<TA, DKMAX, 1, MAXT>(dim3(H, seg.n_items), threads, smem, stream, RET_ARGS);
    if (st) return st;
    const int per_head = DKMAX * (threads / RET_PARTS * 2);
    st = rllm_launch(retention_combine_kernel, dim3(H, n_requests, (per_head + RET_COMBINE_THREADS - 1) / RET_COMBINE_THREADS),
                     dim3(RET_COMBINE_THREADS), 0, stream, (const float*)state, slot_stride, slots, decay, H, per_head, seg);
    if (st) return st;
    return launch_retention_pass<TA, DKMAX, 2, MAXT>(dim3(H, seg.n_items), threads, smem, stream, RET_ARGS);
#undef RET_ARGS
}

// q, k [n, H*dk], v, gate [n, H*dv]: float32 columns of one projection (rows ld apart); gate_kind 0: none
// (gp may be null), 1: silu, 2: sigmoid.  carry needs n_items * H * DKMAX * dvp floats.
RLLM_API int rllm_retention(const float* qp, const float* kp, const float* vp, const float* gp, long long ld,
                            const void* cs_table, int rot, int pairs, float key_scale, const float* decay, float eps,
                            float* state, long long slot_stride, const int* cu_q, const int* slots, void* out,
                            int act_dt, int n_requests, int H, int dk, int dv, int gate_kind, const int* seg_t0,
                            const int* seg_t1, const int* seg_req, const int* seg_flags, const int* req_item0,
                            const int* req_items, int n_items, float* carry, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (dk <= 0 || dk > 256 || dv <= 0 || dv > 256 || H <= 0 || rot < 0 || rot > dk || (rot & 1) || (rot && !cs_table) ||
        (gate_kind && !gp))
        return (int)cudaErrorInvalidValue;
    const int dkmax = ret_dkmax(dk), threads = ret_threads(dv), dvp = threads / RET_PARTS * 2;
    TimeSegments seg = {seg_t0, seg_t1, seg_req, seg_flags, req_item0, req_items, carry, nullptr, n_items};
    if (n_items > 0 && (!seg_t0 || !seg_t1 || !seg_req || !seg_flags || !req_item0 || !req_items || !carry))
        return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)2 * RET_TOK * (2 * dkmax + 2 * dvp) + (size_t)RET_TOK * dvp) * sizeof(float);
#define LAUNCH(TA, DKMAX, MAXT)                                                                                     \
    return launch_retention<TA, DKMAX, MAXT>(n_requests, threads, smem, stream, qp, kp, vp, gp, ld, cs_table, rot,   \
                                             pairs, key_scale, decay, eps, state, slot_stride, cu_q, slots, out, H,  \
                                             dk, dv, gate_kind, seg)
#define BY_D(TA)                                                                                               \
    do {                                                                                                       \
        if (threads > 512) {                                                                                   \
            if (dkmax == 32) { LAUNCH(TA, 32, 1024); }                                                         \
            if (dkmax == 64) { LAUNCH(TA, 64, 1024); }                                                         \
            if (dkmax == 128) { LAUNCH(TA, 128, 1024); }                                                       \
            LAUNCH(TA, 256, 1024);                                                                             \
        }                                                                                                      \
        if (dkmax == 32) { LAUNCH(TA, 32, 512); }                                                              \
        if (dkmax == 64) { LAUNCH(TA, 64, 512); }                                                              \
        if (dkmax == 128) { LAUNCH(TA, 128, 512); }                                                            \
        LAUNCH(TA, 256, 512);                                                                                  \
    } while (0)
    if (act_dt == RLLM_F32) BY_D(float);
    BY_D(bf16);
#undef BY_D
#undef LAUNCH
}

// Floats of a request's retention state for H heads of dk x dv (no device needed).
RLLM_API long long rllm_retention_state_floats(int H, int dk, int dv) {
    return (long long)H * ret_dkmax(dk) * (ret_threads(dv) / RET_PARTS * 2);
}

// ------------------------------------------------------------------ matrix memory with exponential gates (mLSTM)
// One block per (head, request or segment).  Per token, with q, k the head's rows (dk entries), v its
// values (dv entries), and the head's two gate pre-activations x_i, x_f (a bias added here):
//   i = cap * tanh(x_i / cap),  f = logsigmoid(cap * tanh(x_f / cap))            (cap 0: i = x_i, f = logsigmoid(x_f))
//   m' = max(f + m, i);  a = exp(f + m - m'),  b = exp(i - m')
//   S[e][j] = a * S[e][j] + b * k[e] * v[j];   n[e] = a * n[e] + b * k[e]
//   o[j] = q_scale * sum_e q[e] S[e][j] / (max(|q_scale * n . q|, exp(-m')) + 1e-6)
// then o is divided by its root mean square over the head (eps inside the root), multiplied by a weight
// per column and by the gate's activation, and stored in the activation type.  m starts at 0 with S and n
// (a zeroed slot).  The normaliser is carried as one more value column whose "value" is 1 for every
// token, so the thread layout, the chunks of RET_TOK tokens and the slot order are the retention kernel's
// with dv + 1 columns.  The chain of maxima is walked by one thread per chunk (two dependent operations a
// token); the exponentials are then taken by one lane per token.
// Cut along time (TimeSegments): pass 1 runs a segment from an empty memory with m = -infinity and keeps
// (S, n, m) and the sum F of its f; with C = exp(m) S the true memory, C_end = exp(F) C_start + C_local
// and m_end = max(F + m_start, m_local), so   S_end = exp(F + m_start - m_end) S_start + exp(m_local -
// m_end) S_local   (mlstm_combine); pass 2 runs every segment from its true start and writes outputs.
// Scalars behind a head's S, in the slot and in a carry: [0] m, [1] F (carry), [2] m_local (carry).
#define MLSTM_SCALARS 4

template <typename TA, int DKMAX, int PASS, int MAXT>
__global__ void __launch_bounds__(MAXT, (MAXT <= 576 && DKMAX <= 128) ? 2 : 1)
mlstm_kernel(const float* qp, const float* kp, const float* vp, const float* gp, const float* ip, const float* fp,
             long long ld, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
             const float* __restrict__ norm_w, float eps, float* state, long long slot_stride,
             const int* __restrict__ cu_q, const int* __restrict__ slots, TA* out, int H, int dk, int dv, int gate,
             const TimeSegments seg) {
    constexpr int IPT = DKMAX / RET_PARTS;
    extern __shared__ __align__(16) float sm_ml[];
    const int NT = blockDim.x, dvp = NT / RET_PARTS * 2;
    const int stage = RET_TOK * (2 * DKMAX + 2 * dvp + 2);
    float* s_o = sm_ml + 2 * stage;                       // [RET_TOK][dvp]
    float* s_a = s_o + RET_TOK * dvp;                     // a, b, exp(-m'), m' per token of the chunk
    float* s_b = s_a + RET_TOK;
    float* s_em = s_b + RET_TOK;
    float* s_m = s_em + RET_TOK;                          // [RET_TOK + 1]: m before the chunk, then after each token
    const int tid = threadIdx.x, j0 = 2 * (tid / RET_PARTS), part = tid % RET_PARTS;
    const int head = blockIdx.x, item = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    const int r = PASS == 0 ? item : seg.req[item];
    const int t0 = PASS == 0 ? cu_q[r] : seg.t0[item], t1 = PASS == 0 ? cu_q[r + 1] : seg.t1[item];
    const bool first = PASS == 0 || (seg.flags[item] & 1), last = PASS == 0 || (seg.flags[item] & 2);
    if (PASS == 1 && last) return;                        // its end state comes out of pass 2
    const size_t per_S = (size_t)DKMAX * dvp, per_head = per_S + MLSTM_SCALARS;
    float* Sg = state + (size_t)slots[r] * slot_stride + (size_t)head * per_head;
    float S0[IPT], S1[IPT];
    float m_run, f_sum = 0.f;                             // thread 0's: the running maximum, the sum of f
    {
        const int src = first ? item + seg.req_items[r] - 1 : item - 1;
        const float* from = (first && last) ? Sg : seg.carry + ((size_t)src * H + head) * per_head;
#pragma unroll
        for (int ii = 0; ii < IPT; ++ii) {
            S0[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii) * NT + tid];
            S1[ii] = PASS == 1 ? 0.f : from[(size_t)(2 * ii + 1) * NT + tid];
        }
        m_run = PASS == 1 ? -INFINITY : from[per_S];
    }
    const size_t qcol = (size_t)head * dk, vcol = (size_t)head * dv;
    const float ib = i_bias ? i_bias[head] : 0.f, fb = f_bias ? f_bias[head] : 0.f;
    auto issue = [&](int tb, int buf) {
        float* base = sm_ml + buf * stage;
        const int nt = min(RET_TOK, t1 - tb);
        for (int e = tid; e < 2 * RET_TOK * DKMAX; e += NT) {
            const int arr = e / (RET_TOK * DKMAX), rem = e % (RET_TOK * DKMAX), tt = rem / DKMAX, cc = rem % DKMAX;
            if (tt < nt && cc < dk) ret_cp_async4(base + e, (arr ? kp : qp) + (size_t)(tb + tt) * ld + qcol + cc);
            else base[e] = 0.f;
        }
        float* vb = base + 2 * RET_TOK * DKMAX;
        for (int e = tid; e < 2 * RET_TOK * dvp; e += NT) {
            const int arr = e / (RET_TOK * dvp), rem = e % (RET_TOK * dvp), tt = rem / dvp, cc = rem % dvp;
            if (tt < nt && cc < dv && (arr == 0 || gp)) ret_cp_async4(vb + e, (arr ? gp : vp) + (size_t)(tb + tt) * ld + vcol + cc);
            else vb[e] = (arr == 0 && tt < nt && cc == dv) ? 1.f : 0.f;          // the normaliser's column
        }
        float* gb = vb + 2 * RET_TOK * dvp;                                     // the gates' pre-activations
        for (int e = tid; e < 2 * RET_TOK; e += NT) {
            const int arr = e / RET_TOK, tt = e % RET_TOK;
            if (tt < nt) ret_cp_async4(gb + e, (arr ? fp : ip) + (size_t)(tb + tt) * ld + head);
            else gb[e] = 0.f;
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    const int warp = tid >> 5, lane = tid & 31, n_warps = NT >> 5;
    if (t0 < t1) issue(t0, 0);
    int buf = 0;
    for (int tb = t0; tb < t1; tb += RET_TOK, buf ^= 1) {
        const int nt = min(RET_TOK, t1 - tb);
        const bool more = tb + RET_TOK < t1;
        if (more) {
            issue(tb + RET_TOK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        float* s_q = sm_ml + buf * stage;
        float* s_k = s_q + RET_TOK * DKMAX;
        float* s_v = s_k + RET_TOK * DKMAX;
        float* s_g = s_v + RET_TOK * dvp;
        float* s_ig = s_g + RET_TOK * dvp;
        float* s_fg = s_ig + RET_TOK;
        // the gates: one lane per token, then the chain of maxima by one thread, then the exponentials
        if (tid < nt) {
            const float xi = s_ig[tid] + ib, xf = s_fg[tid] + fb;
            s_ig[tid] = cap > 0.f ? cap * tanhf(xi / cap) : xi;
            s_fg[tid] = -softplus_f(-(cap > 0.f ? cap * tanhf(xf / cap) : xf));
        }
        __syncthreads();
        if (tid == 0) {
            s_m[0] = m_run;
            for (int tt = 0; tt < nt; ++tt) {
                m_run = fmaxf(s_fg[tt] + m_run, s_ig[tt]);
                s_m[tt + 1] = m_run;
                f_sum += s_fg[tt];
            }
        }
        __syncthreads();
        if (tid < nt) {
            const float mo = s_m[tid], mn = s_m[tid + 1];
            s_a[tid] = mo == -INFINITY ? 0.f : expf(s_fg[tid] + mo - mn);
            s_b[tid] = expf(s_ig[tid] - mn);
            s_em[tid] = expf(-mn);
        }
        __syncthreads();
        auto token = [&](int tt) {
            const float a = s_a[tt], b = s_b[tt];
            float2 vj = *reinterpret_cast<const float2*>(s_v + tt * dvp + j0);
            vj.x *= b;
            vj.y *= b;
            const float4* q4 = reinterpret_cast<const float4*>(s_q + tt * DKMAX);
            const float4* k4 = reinterpret_cast<const float4*>(s_k + tt * DKMAX);
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int q = 0; q < IPT / 4; ++q) {
                const float4 qq = q4[part + RET_PARTS * q], kk = k4[part + RET_PARTS * q];
#define ML_STEP(Q, K, I, A, B)                                                   \
                S0[I] = a * S0[I] + K * vj.x; S1[I] = a * S1[I] + K * vj.y;      \
                if (PASS != 1) { A += Q * S0[I]; B += Q * S1[I]; }
                ML_STEP(qq.x, kk.x, 4 * q, a0, b0)
                ML_STEP(qq.y, kk.y, 4 * q + 1, a1, b1)
                ML_STEP(qq.z, kk.z, 4 * q + 2, a0, b0)
                ML_STEP(qq.w, kk.w, 4 * q + 3, a1, b1)
#undef ML_STEP
            }
            if (PASS == 1) return;
            float oa = a0 + a1, ob = b0 + b1;
#pragma unroll
            for (int m = 1; m < RET_PARTS; m <<= 1) {
                oa += __shfl_xor_sync(0xffffffffu, oa, m);
                ob += __shfl_xor_sync(0xffffffffu, ob, m);
            }
            if (part == 0) *reinterpret_cast<float2*>(s_o + tt * dvp + j0) = make_float2(oa, ob);
        };
        if (nt == RET_TOK) {
#pragma unroll 2
            for (int tt = 0; tt < RET_TOK; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < nt; ++tt) token(tt);
        }
        __syncthreads();
        for (int tt = warp; PASS != 1 && tt < nt; tt += n_warps) {
            const float nq = s_o[tt * dvp + dv] * q_scale;
            const float inv = q_scale / (fmaxf(fabsf(nq), s_em[tt]) + 1e-6f);
            float ss = 0.f;
            for (int i = lane; i < dv; i += 32) {
                const float o = s_o[tt * dvp + i] * inv;
                ss += o * o;
            }
            const float rs = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
            for (int i = lane; i < dv; i += 32) {
                float v = s_o[tt * dvp + i] * inv * rs;
                if (norm_w) v *= norm_w[vcol + i];
                if (gate == 1) v *= silu_f(s_g[tt * dvp + i]);
                else if (gate == 2) v *= 1.0f / (1.0f + expf(-s_g[tt * dvp + i]));
                out[(size_t)(tb + tt) * H * dv + vcol + i] = from_f<TA>(v);
            }
        }
        __syncthreads();                                  // everyone is done with this buffer, s_o and the gates
    }
    float* to = PASS == 1 ? seg.carry + ((size_t)item * H + head) * per_head : Sg;
    if (PASS != 1 && !last) return;
#pragma unroll
    for (int ii = 0; ii < IPT; ++ii) {
        to[(size_t)(2 * ii) * NT + tid] = S0[ii];
        to[(size_t)(2 * ii + 1) * NT + tid] = S1[ii];
    }
    if (tid == 0) {
        if (PASS == 1) { to[per_S + 1] = f_sum; to[per_S + 2] = m_run; }
        else to[per_S] = m_run;
    }
}

// Between the passes: a request's segments in order, in place; a thread carries one entry of S (or of n).
__global__ void __launch_bounds__(RET_COMBINE_THREADS)
mlstm_combine_kernel(const float* state, long long slot_stride, const int* __restrict__ slots, int H, int per_S,
                     const TimeSegments seg) {
    pdl_wait();
    pdl_launch_dependents();
    const int head = blockIdx.x, r = blockIdx.y;
    const int i = blockIdx.z * RET_COMBINE_THREADS + threadIdx.x;
    const int n = seg.req_items[r], item0 = seg.req_item0[r];
    if (n < 2 || i >= per_S) return;
    const size_t per_head = (size_t)per_S + MLSTM_SCALARS;
    const float* from = state + (size_t)slots[r] * slot_stride + (size_t)head * per_head;
    float S = from[i], m = from[per_S];
    float* start = seg.carry + ((size_t)(item0 + n - 1) * H + head) * per_head;   // the start state, for pass 2
    start[i] = S;
    if (i == 0) start[per_S] = m;
    for (int it = item0; it < item0 + n - 1; ++it) {
        float* C = seg.carry + ((size_t)it * H + head) * per_head;
        const float F = C[per_S + 1], ml = C[per_S + 2];
        const float mn = fmaxf(F + m, ml);
        S = expf(F + m - mn) * S + expf(ml - mn) * C[i];
        m = mn;
        C[i] = S;
        if (i == 0) C[per_S] = m;
    }
}

static inline int mlstm_threads(int dv) { return ret_threads(dv + 1); }

template <typename TA, int DKMAX, int PASS, int MAXT>
static int launch_mlstm_pass(dim3 grid, int threads, size_t smem, cudaStream_t stream, const float* qp, const float* kp,
                             const float* vp, const float* gp, const float* ip, const float* fp, long long ld,
                             const float* i_bias, const float* f_bias, float cap, float q_scale, const float* norm_w,
                             float eps, float* state, long long slot_stride, const int* cu_q, const int* slots, void* out,
                             int H, int dk, int dv, int gate, const TimeSegments& seg) {
    if (smem > 48 * 1024) {
        static size_t raised = 0;
        if (smem > raised) {
            cudaError_t e = cudaFuncSetAttribute(mlstm_kernel<TA, DKMAX, PASS, MAXT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = smem;
        }
    }
    return rllm_launch(mlstm_kernel<TA, DKMAX, PASS, MAXT>, grid, dim3(threads), smem, stream, qp, kp, vp, gp, ip, fp, ld,
                       i_bias, f_bias, cap, q_scale, norm_w, eps, state, slot_stride, cu_q, slots, (TA*)out, H, dk, dv,
                       gate, seg);
}

template <typename TA, int DKMAX, int MAXT>
static int launch_mlstm(int n_requests, int threads, size_t smem, cudaStream_t stream, const float* qp, const float* kp,
                        const float* vp, const float* gp, const float* ip, const float* fp, long long ld,
                        const float* i_bias, const float* f_bias, float cap, float q_scale, const float* norm_w, float eps,
                        float* state, long long slot_stride, const int* cu_q, const int* slots, void* out, int H, int dk,
                        int dv, int gate, const TimeSegments& seg) {
#define ML_ARGS qp, kp, vp, gp, ip, fp, ld, i_bias, f_bias, cap, q_scale, norm_w, eps, state, slot_stride, cu_q, slots, out, H, dk, dv, gate, seg
    if (seg.n_items <= 0)
        return launch_mlstm_pass<TA, DKMAX, 0, MAXT>(dim3(H, n_requests), threads, smem, stream, ML_ARGS);
    int st = launch_mlstm_pass<TA, DKMAX, 1, MAXT>(dim3(H, seg.n_items), threads, smem, stream, ML_ARGS);
    if (st) return st;
    const int per_S = DKMAX * (threads / RET_PARTS * 2);
    st = rllm_launch(mlstm_combine_kernel, dim3(H, n_requests, (per_S + RET_COMBINE_THREADS - 1) / RET_COMBINE_THREADS),
                     dim3(RET_COMBINE_THREADS), 0, stream, (const float*)state, slot_stride, slots, H, per_S, seg);
    if (st) return st;
    return launch_mlstm_pass<TA, DKMAX, 2, MAXT>(dim3(H, seg.n_items), threads, smem, stream, ML_ARGS);
#undef ML_ARGS
}

// ------------------------------------------------------------------ the same recurrence for heads of any size
// Heads too large for the kernel above (keys over 256 entries, values over 254): one block per (head,
// request) walks the request's tokens in order with the memory in the slot itself (global memory, L2 for a
// step's worth): S [dk][dv + 1] row-major, whose column dv is the normaliser, then four floats of which the
// first is m.  A thread owns every 256th column: S[e][j] = a S[e][j] + k[e] (b v[j]), o[j] += q[e] S[e][j].
// Slow (the state crosses L2 once a token) and exact in the same order of operations; not cut along time.
template <typename TA>
__global__ void __launch_bounds__(256)
mlstm_generic_kernel(const float* qp, const float* kp, const float* vp, const float* gp, const float* ip, const float* fp,
                     long long ld, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                     float q_scale, const float* __restrict__ norm_w, float eps, float* state, long long slot_stride,
                     const int* __restrict__ cu_q, const int* __restrict__ slots, TA* out, int H, int dk, int dv, int gate) {
    extern __shared__ float sm_g[];
    __shared__ float red[33];
    __shared__ float s_gate[3];                           // a, b, exp(-m')
    const int dvp = dv + 1;
    float* s_q = sm_g;                                    // [dk]
    float* s_k = s_q + dk;                                // [dk]
    float* s_o = s_k + dk;                                // [dvp]
    const int tid = threadIdx.x, head = blockIdx.x, r = blockIdx.y;
    pdl_wait();
    pdl_launch_dependents();
    const size_t per_S = (size_t)dk * dvp;
    float* S = state + (size_t)slots[r] * slot_stride + (size_t)head * (per_S + MLSTM_SCALARS);
    float m_run = S[per_S];
    const size_t qcol = (size_t)head * dk, vcol = (size_t)head * dv;
    const float ib = i_bias ? i_bias[head] : 0.f, fb = f_bias ? f_bias[head] : 0.f;
    for (int t = cu_q[r]; t < cu_q[r + 1]; ++t) {
        for (int e = tid; e < dk; e += blockDim.x) {
            s_q[e] = qp[(size_t)t * ld + qcol + e];
            s_k[e] = kp[(size_t)t * ld + qcol + e];
        }
        if (tid == 0) {
            const float xi = ip[(size_t)t * ld + head] + ib, xf = fp[(size_t)t * ld + head] + fb;
            const float ig = cap > 0.f ? cap * tanhf(xi / cap) : xi;
            const float fg = -softplus_f(-(cap > 0.f ? cap * tanhf(xf / cap) : xf));
            const float mn = fmaxf(fg + m_run, ig);
            s_gate[0] = expf(fg + m_run - mn);
            s_gate[1] = expf(ig - mn);
            s_gate[2] = expf(-mn);
            m_run = mn;
        }
        __syncthreads();
        const float a = s_gate[0], b = s_gate[1];
        for (int j = tid; j < dvp; j += blockDim.x) {
            const float vj = (j < dv ? vp[(size_t)t * ld + vcol + j] : 1.f) * b;
            float acc = 0.f;
            for (int e = 0; e < dk; ++e) {
                const float sv = a * S[(size_t)e * dvp + j] + s_k[e] * vj;
                S[(size_t)e * dvp + j] = sv;
                acc += s_q[e] * sv;
            }
            s_o[j] = acc;
        }
        __syncthreads();
        const float nq = s_o[dv] * q_scale;
        const float inv = q_scale / (fmaxf(fabsf(nq), s_gate[2]) + 1e-6f);
        float ss = 0.f;
        for (int j = tid; j < dv; j += blockDim.x) {
            const float o = s_o[j] * inv;
            ss += o * o;
        }
        ss = block_sum(ss, red);
        const float rs = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int j = tid; j < dv; j += blockDim.x) {
            float v = s_o[j] * inv * rs;
            if (norm_w) v *= norm_w[vcol + j];
            if (gate) {
                const float gz = gp[(size_t)t * ld + vcol + j];
                v *= gate == 1 ? silu_f(gz) : 1.0f / (1.0f + expf(-gz));
            }
            out[(size_t)t * H * dv + vcol + j] = from_f<TA>(v);
        }
        __syncthreads();                                  // s_q, s_k, s_o and the gates are free again
    }
    if (tid == 0) S[per_S] = m_run;
}

static inline bool mlstm_fits_fast(int dk, int dv) { return dk <= 256 && dv <= 254; }

// q, k [n, H*dk], v, gate [n, H*dv], the gates' pre-activations ip, fp [n, H]: float32 columns of one
// projection (rows ld apart); i_bias, f_bias [H] or null; norm_w [H*dv] or null; gate_kind 0: none, 1: silu,
// 2: sigmoid.  carry needs n_items * H * (DKMAX * dvp + 4) floats.
RLLM_API int rllm_mlstm(const float* qp, const float* kp, const float* vp, const float* gp, const float* ip,
                        const float* fp, long long ld, const float* i_bias, const float* f_bias, float cap, float q_scale,
                        const float* norm_w, float eps, float* state, long long slot_stride, const int* cu_q,
                        const int* slots, void* out, int act_dt, int n_requests, int H, int dk, int dv, int gate_kind,
                        const int* seg_t0, const int* seg_t1, const int* seg_req, const int* seg_flags,
                        const int* req_item0, const int* req_items, int n_items, float* carry, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (dk <= 0 || dv <= 0 || H <= 0 || cap < 0.f || (gate_kind && !gp) || !ip || !fp) return (int)cudaErrorInvalidValue;
    if (!mlstm_fits_fast(dk, dv)) {
        const size_t smem_g = ((size_t)2 * dk + dv + 1) * sizeof(float);
        if (smem_g > 48 * 1024) return (int)cudaErrorInvalidValue;
        if (act_dt == RLLM_F32)
            return rllm_launch(mlstm_generic_kernel<float>, dim3(H, n_requests), dim3(256), smem_g, stream, qp, kp, vp, gp, ip,
                               fp, ld, i_bias, f_bias, cap, q_scale, norm_w, eps, state, slot_stride, cu_q, slots,
                               (float*)out, H, dk, dv, gate_kind);
        return rllm_launch(mlstm_generic_kernel<bf16>, dim3(H, n_requests), dim3(256), smem_g, stream, qp, kp, vp, gp, ip, fp,
                           ld, i_bias, f_bias, cap, q_scale, norm_w, eps, state, slot_stride, cu_q, slots, (bf16*)out, H, dk,
                           dv, gate_kind);
    }
    const int dkmax = ret_dkmax(dk), threads = mlstm_threads(dv), dvp = threads / RET_PARTS * 2;
    TimeSegments seg = {seg_t0, seg_t1, seg_req, seg_flags, req_item0, req_items, carry, nullptr, n_items};
    if (n_items > 0 && (!seg_t0 || !seg_t1 || !seg_req || !seg_flags || !req_item0 || !req_items || !carry))
        return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)2 * RET_TOK * (2 * dkmax + 2 * dvp + 2) + (size_t)RET_TOK * dvp + 4 * RET_TOK + 4) * sizeof(float);
#define LAUNCH(TA, DKMAX, MAXT)                                                                                    \
    return launch_mlstm<TA, DKMAX, MAXT>(n_requests, threads, smem, stream, qp, kp, vp, gp, ip, fp, ld, i_bias, f_bias, \
                                         cap, q_scale, norm_w, eps, state, slot_stride, cu_q, slots, out, H, dk, dv, \
                                         gate_kind, seg)
    // blocks of up to 576 threads (value heads up to 142 entries and the normaliser's column) are compiled for
    // two blocks an SM: 128 value columns take 544 threads, one warp more than 512
#define BY_D(TA)                                                                                               \
    do {                                                                                                       \
        if (threads > 576) {                                                                                   \
            if (dkmax == 32) { LAUNCH(TA, 32, 1024); }                                                         \
            if (dkmax == 64) { LAUNCH(TA, 64, 1024); }                                                         \
            if (dkmax == 128) { LAUNCH(TA, 128, 1024); }                                                       \
            LAUNCH(TA, 256, 1024);                                                                             \
        }                                                                                                      \
        if (dkmax == 32) { LAUNCH(TA, 32, 576); }                                                              \
        if (dkmax == 64) { LAUNCH(TA, 64, 576); }                                                              \
        if (dkmax == 128) { LAUNCH(TA, 128, 576); }                                                            \
        LAUNCH(TA, 256, 576);                                                                                  \
    } while (0)
    if (act_dt == RLLM_F32) BY_D(float);
    BY_D(bf16);
#undef BY_D
#undef LAUNCH
}

// Floats of a request's mLSTM state for H heads of dk x dv (no device needed).
RLLM_API long long rllm_mlstm_state_floats(int H, int dk, int dv) {
    if (!mlstm_fits_fast(dk, dv)) return (long long)H * ((long long)dk * (dv + 1) + MLSTM_SCALARS);
    return (long long)H * ((long long)ret_dkmax(dk) * (mlstm_threads(dv) / RET_PARTS * 2) + MLSTM_SCALARS);
}

RLLM_PACKED(rllm_conv_silu)
RLLM_PACKED(rllm_mlstm)
RLLM_PACKED(rllm_retention)
RLLM_PACKED(rllm_selective_scan)
RLLM_PACKED(rllm_token_shift)
RLLM_PACKED(rllm_wkv)
