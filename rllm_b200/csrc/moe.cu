// Routed feed-forward experts: the router's choice, and the experts' products for steps of few rows.
// float32 arithmetic for everything the router does (accurate expf); products accumulate in float32 in a
// fixed order, so a token's result does not depend on the batch around it.
//
//   moe_route        per token: scores from the router's logits (sigmoid, or softmax over all experts),
//                    choice scores = scores + correction; experts form equal groups of neighbours, a
//                    group's score is the sum of its `group_best` largest choice scores, only the
//                    `keep_groups` best groups can be chosen from; the `top_k` largest choice scores win
//                    (ties: the lower index); weights = the winners' scores (without the correction),
//                    divided by their sum + weight_eps when `normalize`, times route_scale.
//   moe_pairs_gate_up  act[pair, f] = glu(Wg[e] . h[t], Wu[e] . h[t]) for every (token, chosen expert) pair:
//                    a block per (pair, tile of columns), a warp per column, the token's row in shared memory.
//   moe_pairs_down   out[t, c] = sum_j weight[t, j] * (Wd[e_j][c, :] . act[t * top_k + j, :]) in the order of j,
//                    plus shared[t, c] * sigmoid(shared_gate[t]) when a shared expert's output is given.
//   moe_sort         pairs counted per expert, offsets, and each pair's place in expert order (a stable
//                    counting sort by one block); moe_gather_rows copies the tokens' rows into that order
//                    and moe_combine adds a token's expert outputs back in the order of j.
#include "common.cuh"
#include <math.h>

#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 32

__global__ void __launch_bounds__(32)
moe_route_kernel(const float* logits, long long ld, const float* __restrict__ correction, int* idx, float* weight,
                 int E, int top_k, int n_groups, int keep_groups, int group_best, int softmax, int normalize,
                 float weight_eps, float route_scale) {
    __shared__ float s_score[MOE_MAX_EXPERTS];
    __shared__ float s_choice[MOE_MAX_EXPERTS];
    __shared__ float s_group[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* z = logits + (size_t)t * ld;
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float p = expf(z[e] - m);
            s_score[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) s_score[e] /= sum;
    } else {
        for (int e = lane; e < E; e += 32) s_score[e] = 1.0f / (1.0f + expf(-z[e]));
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) s_choice[e] = s_score[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    const int per = E / n_groups;
    if (keep_groups < n_groups) {
        // a group's score: the sum of its largest choice scores (one lane per group, in index order)
        for (int g = lane; g < n_groups; g += 32) {
            float sum = 0.f;
            float last = INFINITY;
            int last_i = -1;
            for (int b = 0; b < group_best && b < per; ++b) {
                float best = -INFINITY;
                int bi = -1;
                for (int i = 0; i < per; ++i) {
                    const float c = s_choice[g * per + i];
                    // candidates: strictly below the last pick, or equal to it with a larger index
                    const bool free_ = c < last || (c == last && i > last_i);
                    if (free_ && (c > best || bi < 0)) { best = c; bi = i; }
                }
                if (bi < 0) break;
                sum += best;
                last = best;
                last_i = bi;
            }
            s_group[g] = sum;
        }
        __syncwarp();
        // keep the best groups: a group is kept if fewer than keep_groups groups beat it
        for (int g = lane; g < n_groups; g += 32) {
            int beat = 0;
            const float mine = s_group[g];
            for (int o = 0; o < n_groups; ++o) {
                const float other = s_group[o];
                beat += (other > mine || (other == mine && o < g)) ? 1 : 0;
            }
            if (beat >= keep_groups)
                for (int i = 0; i < per; ++i) s_choice[g * per + i] = -INFINITY;
        }
        __syncwarp();
    }
    // the top_k largest choice scores, one after the other; ties go to the lower index
    float wsum = 0.f;
    for (int j = 0; j < top_k; ++j) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = s_choice[e];
            if (c > best) { best = c; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (bi >= E) bi = 0;                                 // nothing left to choose from (never with valid sizes)
        const float s = s_score[bi];
        wsum += s;
        if (lane == 0) {
            s_choice[bi] = -INFINITY;
            idx[(size_t)t * top_k + j] = bi;
            weight[(size_t)t * top_k + j] = s;               // divided below
        }
        __syncwarp();
    }
    __syncwarp();
    const float mul = (normalize ? 1.0f / (wsum + weight_eps) : 1.0f) * route_scale;
    for (int j = lane; j < top_k; j += 32) weight[(size_t)t * top_k + j] *= mul;
}

RLLM_API int rllm_moe_route(const float* logits, long long ld, const float* correction, int* idx, float* weight, int n,
                            int E, int top_k, int n_groups, int keep_groups, int group_best, int softmax, int normalize,
                            float weight_eps, float route_scale, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS || top_k <= 0 || top_k > E || n_groups <= 0 || E % n_groups || keep_groups <= 0 ||
        keep_groups > n_groups || group_best <= 0 || ld < E)
        return (int)cudaErrorInvalidValue;
    return rllm_launch(moe_route_kernel, dim3(n), dim3(32), 0, stream, logits, ld, correction, idx, weight, E, top_k,
                       n_groups, keep_groups, group_best, softmax, normalize, weight_eps, route_scale);
}

// ------------------------------------------------------------------ experts, pair by pair
__device__ __forceinline__ float dot_row(const float* w, const float* x, int k, int lane) {
    float acc = 0.f;
    for (int i = lane; i < k; i += 32) acc += w[i] * x[i];
    return acc;
}
__device__ __forceinline__ float dot_row(const bf16* w, const float* x, int k, int lane) {
    float acc = 0.f;
    if ((k & 7) == 0 && ((uintptr_t)w & 15) == 0) {
        for (int i = lane * 8; i < k; i += 256) {
            const uint4 u = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(p[q]);
                acc += f.x * x[i + 2 * q] + f.y * x[i + 2 * q + 1];
            }
        }
    } else {
        for (int i = lane; i < k; i += 32) acc += __bfloat162float(w[i]) * x[i];
    }
    return acc;
}

#define MOE_COLS 32      // columns per block (8 warps, 4 columns a warp)

// h [n, d]; w_gu [E][2F][d] (gate rows, then up rows); act [n * top_k, F]
template <typename T>
__global__ void __launch_bounds__(256)
moe_pairs_gate_up_kernel(const T* h, const T* __restrict__ w_gu, const int* idx, T* act, int top_k, int d, int F,
                         GluForm glu) {
    extern __shared__ float s_h[];
    pdl_wait();
    pdl_launch_dependents();
    const int pair = blockIdx.x, t = pair / top_k, e = idx[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s_h[i] = to_f<T>(h[(size_t)t * d + i]);
    __syncthreads();
    const T* wg = w_gu + (size_t)e * 2 * F * d;
    for (int c = warp; c < MOE_COLS; c += 8) {
        const int f = blockIdx.y * MOE_COLS + c;
        if (f >= F) break;
        float g = dot_row(wg + (size_t)f * d, s_h, d, lane);
        float u = dot_row(wg + (size_t)(F + f) * d, s_h, d, lane);
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) {
            if (glu.limit > 0.f) {
                g = fminf(g, glu.limit);
                u = fminf(fmaxf(u, -glu.limit), glu.limit);
            }
            act[(size_t)pair * F + f] = from_f<T>(g / (1.0f + expf(-glu.alpha * g)) * (u + glu.shift));
        }
    }
}

// act [n * top_k, F]; w_down [E][d][F]; out [n, d] float32; shared [n, d] float32 or null; gate: logits, one per token
template <typename T>
__global__ void __launch_bounds__(256)
moe_pairs_down_kernel(const T* act, const T* __restrict__ w_down, const int* idx, const float* weight, float* out,
                      const float* shared, const float* gate, long long ld_gate, int top_k, int d, int F) {
    extern __shared__ float s_a[];          // [top_k][F]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top_k * F; i += blockDim.x) s_a[i] = to_f<T>(act[(size_t)t * top_k * F + i]);
    __syncthreads();
    const float sg = (shared && gate) ? 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate])) : 1.0f;
    for (int c = warp; c < MOE_COLS; c += 8) {
        const int col = blockIdx.y * MOE_COLS + c;
        if (col >= d) break;
        float sum = 0.f;
        for (int j = 0; j < top_k; ++j) {
            const int e = idx[(size_t)t * top_k + j];
            const float v = warp_sum(dot_row(w_down + ((size_t)e * d + col) * F, s_a + (size_t)j * F, F, lane));
            sum += weight[(size_t)t * top_k + j] * v;
        }
        if (lane == 0) out[(size_t)t * d + col] = sum + (shared ? shared[(size_t)t * d + col] * sg : 0.f);
    }
}

RLLM_API int rllm_moe_pairs_gate_up(const void* h, const void* w_gu, int dt, const int* idx, void* act, int n, int top_k,
                                    int d, int F, float limit, float alpha, float shift, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || F <= 0 || top_k <= 0 || (size_t)d * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid(n * top_k, (F + MOE_COLS - 1) / MOE_COLS);
    const GluForm glu = {limit, alpha, shift};
    if (dt == RLLM_F32)
        return rllm_launch(moe_pairs_gate_up_kernel<float>, grid, dim3(256), (size_t)d * sizeof(float), stream,
                           (const float*)h, (const float*)w_gu, idx, (float*)act, top_k, d, F, glu);
    return rllm_launch(moe_pairs_gate_up_kernel<bf16>, grid, dim3(256), (size_t)d * sizeof(float), stream, (const bf16*)h,
                       (const bf16*)w_gu, idx, (bf16*)act, top_k, d, F, glu);
}

RLLM_API int rllm_moe_pairs_down(const void* act, const void* w_down, int dt, const int* idx, const float* weight,
                                 float* out, const float* shared, const float* gate, long long ld_gate, int n, int top_k,
                                 int d, int F, cudaStream_t stream) {
    if (n <= 0) return 0;
    const size_t smem = (size_t)top_k * F * sizeof(float);
    if (d <= 0 || F <= 0 || top_k <= 0 || smem > 96 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid(n, (d + MOE_COLS - 1) / MOE_COLS);
    if (smem > 48 * 1024) {
        static size_t raised_f = 0, raised_b = 0;
        size_t& raised = dt == RLLM_F32 ? raised_f : raised_b;
        if (smem > raised) {
            cudaError_t e = dt == RLLM_F32
                ? cudaFuncSetAttribute(moe_pairs_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                : cudaFuncSetAttribute(moe_pairs_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            raised = smem;
        }
    }
    if (dt == RLLM_F32)
        return rllm_launch(moe_pairs_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)act,
                           (const float*)w_down, idx, weight, out, shared, gate, ld_gate, top_k, d, F);
    return rllm_launch(moe_pairs_down_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)act, (const bf16*)w_down,
                       idx, weight, out, shared, gate, ld_gate, top_k, d, F);
}

// ------------------------------------------------------------------ many rows: pairs in expert order
// One block.  counts[e], offsets[e] (E + 1 entries) and place[pair]: the pair's row among all pairs sorted
// by expert, pairs of one expert in pair order (stable), so the order never depends on scheduling.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* idx, int n_pairs, int E, int* offsets, int* place) {
    __shared__ int s_count[MOE_MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    for (int e = tid; e <= E; e += blockDim.x) s_count[e] = 0;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) atomicAdd(&s_count[idx[p]], 1);
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = s_count[e];
            s_count[e] = run;
            offsets[e] = run;
            run += c;
        }
        offsets[E] = run;
    }
    __syncthreads();
    // a thread per expert walks the pairs in order: stable, and no atomics on the places
    for (int e = tid; e < E; e += blockDim.x) {
        if (offsets[e + 1] == offsets[e]) continue;
        int at = offsets[e];
        for (int p = 0; p < n_pairs; ++p)
            if (idx[p] == e) place[p] = at++;
    }
}

RLLM_API int rllm_moe_sort(const int* idx, int n_pairs, int E, int* offsets, int* place, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS) return (int)cudaErrorInvalidValue;
    return rllm_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, idx, n_pairs, E, offsets, place);
}

// rows[place[pair]] = h[pair / top_k]
template <typename T>
__global__ void moe_gather_rows_kernel(const T* h, const int* place, T* rows, int top_k, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int pair = blockIdx.x;
    const T* src = h + (size_t)(pair / top_k) * d;
    T* dst = rows + (size_t)place[pair] * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
}

RLLM_API int rllm_moe_gather_rows(const void* h, int dt, const int* place, void* rows, int n_pairs, int top_k, int d,
                                  cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (dt == RLLM_F32)
        return rllm_launch(moe_gather_rows_kernel<float>, dim3(n_pairs), dim3(128), 0, stream, (const float*)h, place,
                           (float*)rows, top_k, d);
    return rllm_launch(moe_gather_rows_kernel<bf16>, dim3(n_pairs), dim3(128), 0, stream, (const bf16*)h, place,
                       (bf16*)rows, top_k, d);
}

// out[t] = sum_j weight[t, j] * y[place[t * top_k + j]] (+ shared[t] * sigmoid(gate[t]))
__global__ void moe_combine_kernel(const float* y, const int* place, const float* weight, float* out, const float* shared,
                                   const float* gate, long long ld_gate, int top_k, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float sg = (shared && gate) ? 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate])) : 1.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float sum = 0.f;
        for (int j = 0; j < top_k; ++j)
            sum += weight[(size_t)t * top_k + j] * y[(size_t)place[(size_t)t * top_k + j] * d + i];
        out[(size_t)t * d + i] = sum + (shared ? shared[(size_t)t * d + i] * sg : 0.f);
    }
}

RLLM_API int rllm_moe_combine(const float* y, const int* place, const float* weight, float* out, const float* shared,
                              const float* gate, long long ld_gate, int n, int top_k, int d, cudaStream_t stream) {
    if (n <= 0) return 0;
    return rllm_launch(moe_combine_kernel, dim3(n), dim3(d >= 1024 ? 256 : 128), 0, stream, y, place, weight, out, shared,
                       gate, ld_gate, top_k, d);
}

RLLM_PACKED(rllm_moe_route)
RLLM_PACKED(rllm_moe_pairs_gate_up)
RLLM_PACKED(rllm_moe_pairs_down)
RLLM_PACKED(rllm_moe_sort)
RLLM_PACKED(rllm_moe_gather_rows)
RLLM_PACKED(rllm_moe_combine)
