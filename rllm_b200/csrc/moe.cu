// Routed feed-forward experts: the router's choice, and the experts' products for steps of few rows.
// float32 arithmetic for everything the router does (accurate expf); products accumulate in float32 in a
// fixed order, so a token's result does not depend on the batch around it.
//
//   moe_route        per token: scores from the router's logits (plus a stored bias per expert, if any; sigmoid, or softmax over all experts),
//                    choice scores = scores + correction; experts form equal groups of neighbours, a
//                    group's score is the sum of its `group_best` largest choice scores, only the
//                    `keep_groups` best groups can be chosen from; the `top_k` largest choice scores win
//                    (ties: the lower index); weights = the winners' scores (without the correction),
//                    divided by their sum + weight_eps when `normalize`, times route_scale.
//   moe_pairs_gate_up  act[pair, f] = glu(Wg[e] . h[t], Wu[e] . h[t]) for every (token, chosen expert) pair:
//                    a block per (pair, tile of columns), the token's row in shared memory; a warp runs the
//                    gate and up rows of four columns side by side (eight 16-byte loads in flight per lane).
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
                 float weight_eps, float route_scale, const float* __restrict__ bias) {
    __shared__ float s_score[MOE_MAX_EXPERTS];
    __shared__ float s_choice[MOE_MAX_EXPERTS];
    __shared__ float s_group[MOE_MAX_EXPERTS];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x;
    const float* z = logits + (size_t)t * ld;
    if (bias) {                                              // the logits with their bias, staged in s_group
        for (int e = lane; e < E; e += 32) s_group[e] = z[e] + bias[e];
        __syncwarp();
        z = s_group;
    }
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
    __syncwarp();                                            // (s_group is free again: z is not read below)
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
                            float weight_eps, float route_scale, const float* bias, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS || top_k <= 0 || top_k > E || n_groups <= 0 || E % n_groups || keep_groups <= 0 ||
        keep_groups > n_groups || group_best <= 0 || ld < E)
        return (int)cudaErrorInvalidValue;
    return rllm_launch(moe_route_kernel, dim3(n), dim3(32), 0, stream, logits, ld, correction, idx, weight, E, top_k,
                       n_groups, keep_groups, group_best, softmax, normalize, weight_eps, route_scale, bias);
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

// 8 bfloat16 weights (one 16-byte load) against 8 floats
__device__ __forceinline__ float dot8(const uint4& u, const float4& xa, const float4& xb) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]),
                 e = __bfloat1622float2(p[3]);
    return a.x * xa.x + a.y * xa.y + b.x * xa.z + b.y * xa.w + c.x * xb.x + c.y * xb.y + e.x * xb.z + e.y * xb.w;
}
__device__ __forceinline__ bool rows_vec_ok(const void* w, int k) { return (k & 7) == 0 && ((uintptr_t)w & 15) == 0; }

// h [n, d]; w_gu [E][2F][d] (gate rows, then up rows); act [n * top_k, F]
template <typename T>
__global__ void __launch_bounds__(256)
moe_pairs_gate_up_kernel(const T* h, const T* __restrict__ w_gu, const int* idx, T* act, int top_k, int d, int F,
                         GluForm glu) {
    extern __shared__ __align__(16) float s_h[];
    pdl_wait();
    pdl_launch_dependents();
    const int pair = blockIdx.x, t = pair / top_k, e = idx[pair];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s_h[i] = to_f<T>(h[(size_t)t * d + i]);
    __syncthreads();
    const T* wg = w_gu + (size_t)e * 2 * F * d;
    if constexpr (sizeof(T) == 2) {
        if (rows_vec_ok(wg, d)) {
            // the warp's four columns at once: eight rows (gate and up), a 16-byte load of each in flight per lane
            const T* rows[8];
            int fcol[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                fcol[q] = blockIdx.y * MOE_COLS + warp + 8 * q;
                const int fc = min(fcol[q], F - 1);
                rows[q] = wg + (size_t)fc * d;
                rows[4 + q] = wg + (size_t)(F + fc) * d;
            }
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int i = lane * 8; i < d; i += 256) {
                uint4 u[8];
#pragma unroll
                for (int r = 0; r < 8; ++r) u[r] = *reinterpret_cast<const uint4*>(rows[r] + i);
                const float4 xa = *reinterpret_cast<const float4*>(s_h + i), xb = *reinterpret_cast<const float4*>(s_h + i + 4);
#pragma unroll
                for (int r = 0; r < 8; ++r) acc[r] += dot8(u[r], xa, xb);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) acc[r] = warp_sum(acc[r]);
            if (lane == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (fcol[q] >= F) continue;
                    float g = acc[q], u = acc[4 + q];
                    if (glu.limit > 0.f) {
                        g = fminf(g, glu.limit);
                        u = fminf(fmaxf(u, -glu.limit), glu.limit);
                    }
                    act[(size_t)pair * F + fcol[q]] = from_f<T>(g / (1.0f + expf(-glu.alpha * g)) * (u + glu.shift));
                }
            }
            return;
        }
    }
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
    extern __shared__ __align__(16) float s_a[];          // [top_k][F]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top_k * F; i += blockDim.x) s_a[i] = to_f<T>(act[(size_t)t * top_k * F + i]);
    __syncthreads();
    const float sg = (shared && gate) ? 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate])) : 1.0f;
    if constexpr (sizeof(T) == 2) {
        if (rows_vec_ok(w_down, F)) {
            // two of the warp's columns and four of the token's experts at once: eight 16-byte loads in flight per
            // lane; a lane weights its partial sums in the order of j, one warp sum per column
            for (int q0 = 0; q0 < 4; q0 += 2) {
                const int col0 = blockIdx.y * MOE_COLS + warp + 8 * q0, col1 = col0 + 8;
                if (col0 >= d) break;
                const int c1 = min(col1, d - 1);
                float tot0 = 0.f, tot1 = 0.f;
                for (int j0 = 0; j0 < top_k; j0 += 4) {
                    const T* rows[8];
                    const float* xs[4];
                    float wj[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int j = min(j0 + jj, top_k - 1);
                        const int e = idx[(size_t)t * top_k + j];
                        wj[jj] = j0 + jj < top_k ? weight[(size_t)t * top_k + j] : 0.f;
                        rows[jj] = w_down + ((size_t)e * d + col0) * F;
                        rows[4 + jj] = w_down + ((size_t)e * d + c1) * F;
                        xs[jj] = s_a + (size_t)j * F;
                    }
                    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    for (int i = lane * 8; i < F; i += 256) {
                        uint4 u[8];
#pragma unroll
                        for (int r = 0; r < 8; ++r) u[r] = *reinterpret_cast<const uint4*>(rows[r] + i);
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float4 xa = *reinterpret_cast<const float4*>(xs[jj] + i),
                                         xb = *reinterpret_cast<const float4*>(xs[jj] + i + 4);
                            acc[jj] += dot8(u[jj], xa, xb);
                            acc[4 + jj] += dot8(u[4 + jj], xa, xb);
                        }
                    }
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        tot0 += wj[jj] * acc[jj];
                        tot1 += wj[jj] * acc[4 + jj];
                    }
                }
                tot0 = warp_sum(tot0);
                tot1 = warp_sum(tot1);
                if (lane == 0) {
                    out[(size_t)t * d + col0] = tot0 + (shared ? shared[(size_t)t * d + col0] * sg : 0.f);
                    if (col1 < d) out[(size_t)t * d + col1] = tot1 + (shared ? shared[(size_t)t * d + col1] * sg : 0.f);
                }
            }
            return;
        }
    }
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

// ------------------------------------------------------------------ experts, expert by expert (bfloat16, few rows)
// The same products on the tensor cores, with a block per (expert, tile of columns): the block lists the pairs
// that chose its expert (in pair order) and runs them eight at a time as the n side of mma.sync m16n8k16, the
// expert's rows as the m side.  An expert's matrices are read once per eight of its tokens, straight from
// global memory into the A fragments (no conversion, no shared memory); an expert that nobody chose costs a
// scan of idx.  A token's sums are formed in the same order whatever else the list holds.
//
// Fragments without ldmatrix: within a step of 32 k, lane (g = lane / 4, c = lane % 4) loads the 16 bytes
// [8c, 8c + 8) of rows g and g + 8 and of token g.  A dot product does not care in which order k is walked as
// long as both operands walk alike, so the first four bytes of each load serve as the k pair (2c, 2c + 1) of
// one mma, the next four as its pair (2c + 8, 2c + 9), and the second half of the load feeds a second mma.
#define MOE_MT 8         // tokens of an expert side by side (n of the mma)
#define MOE_LIST 1024    // pairs of one expert a block can list (a token chooses an expert once: rows of the step)

__device__ __forceinline__ int list_expert_pairs(const int* idx, int n_pairs, int e, int* s_list, int* s_n) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        int cnt = 0;
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool mine = p < n_pairs && idx[p] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            const int at = cnt + __popc(m & ((1u << lane) - 1u));
            if (mine && at < MOE_LIST) s_list[at] = p;
            cnt += __popc(m);
        }
        if (lane == 0) *s_n = min(cnt, MOE_LIST);
    }
    __syncthreads();
    return *s_n;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Rows lo (this lane's row g) and hi (row g + 8) of k entries against the lane's token row x: acc[0], acc[1] = row g
// times tokens 2c and 2c + 1, acc[2], acc[3] = row g + 8 times the same.  Four steps of 32 k in flight (eight
// 16-byte loads of weights a lane); two accumulators take turns and are added at the end.
__device__ __forceinline__ void rows16_times_tokens8(const bf16* lo, const bf16* hi, const bf16* x, int k, int c,
                                                     float (&acc)[4]) {
    float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
    const int off = 8 * c;
    int k0 = 0;
    for (; k0 + 128 <= k; k0 += 128) {
        uint4 v[4], w[4], xb[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            v[s] = *reinterpret_cast<const uint4*>(lo + k0 + 32 * s + off);
            w[s] = *reinterpret_cast<const uint4*>(hi + k0 + 32 * s + off);
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) xb[s] = *reinterpret_cast<const uint4*>(x + k0 + 32 * s + off);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            mma_16816(a0, v[s].x, w[s].x, v[s].y, w[s].y, xb[s].x, xb[s].y);
            mma_16816(a1, v[s].z, w[s].z, v[s].w, w[s].w, xb[s].z, xb[s].w);
        }
    }
    for (; k0 < k; k0 += 32) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u), w = v, xb = v;
        if (k0 + off < k) {
            v = *reinterpret_cast<const uint4*>(lo + k0 + off);
            w = *reinterpret_cast<const uint4*>(hi + k0 + off);
            xb = *reinterpret_cast<const uint4*>(x + k0 + off);
        }
        mma_16816(a0, v.x, w.x, v.y, w.y, xb.x, xb.y);
        mma_16816(a1, v.z, w.z, v.w, w.w, xb.z, xb.w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = a0[i] + a1[i];
}

// 4 warps; a warp takes 8 columns: their gate rows are rows 0..7 of its mma, their up rows rows 8..15, so a
// lane ends up with gate and up of one column for two tokens.
__global__ void __launch_bounds__(128)
moe_expert_gate_up_kernel(const bf16* h, const bf16* __restrict__ w_gu, const int* idx, bf16* act, int n_pairs, int top_k,
                          int d, int F, GluForm glu) {
    __shared__ int s_list[MOE_LIST];
    __shared__ int s_n;
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int cnt = list_expert_pairs(idx, n_pairs, e, s_list, &s_n);
    if (cnt == 0) return;
    const int f = blockIdx.y * MOE_COLS + warp * 8 + g;
    const bf16* wg = w_gu + (size_t)e * 2 * F * d;
    const bf16* lo = wg + (size_t)min(f, F - 1) * d;
    const bf16* hi = wg + (size_t)(F + min(f, F - 1)) * d;
    for (int c0 = 0; c0 < cnt; c0 += MOE_MT) {
        const int mine = s_list[min(c0 + g, cnt - 1)];                     // the token this lane loads for the n side
        float acc[4];
        rows16_times_tokens8(lo, hi, h + (size_t)(mine / top_k) * d, d, c, acc);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int at = c0 + 2 * c + q;
            if (at >= cnt || f >= F) continue;
            float gv = acc[q], uv = acc[2 + q];
            if (glu.limit > 0.f) {
                gv = fminf(gv, glu.limit);
                uv = fminf(fmaxf(uv, -glu.limit), glu.limit);
            }
            act[(size_t)s_list[at] * F + f] = from_f<bf16>(gv / (1.0f + expf(-glu.alpha * gv)) * (uv + glu.shift));
        }
    }
}

#define MOE_DOWN_COLS 64     // columns per block of the down product (4 warps, 16 columns a warp)

// y[pair, col] = Wd[e][col, :] . act[pair, :] for the pairs of the block's expert; moe_combine weights and adds them
__global__ void __launch_bounds__(128)
moe_expert_down_kernel(const bf16* act, const bf16* __restrict__ w_down, const int* idx, float* y, int n_pairs, int d,
                       int F) {
    __shared__ int s_list[MOE_LIST];
    __shared__ int s_n;
    pdl_wait();
    pdl_launch_dependents();
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int cnt = list_expert_pairs(idx, n_pairs, e, s_list, &s_n);
    if (cnt == 0) return;
    const int col_lo = blockIdx.y * MOE_DOWN_COLS + warp * 16 + g, col_hi = col_lo + 8;
    const bf16* lo = w_down + ((size_t)e * d + min(col_lo, d - 1)) * F;
    const bf16* hi = w_down + ((size_t)e * d + min(col_hi, d - 1)) * F;
    for (int c0 = 0; c0 < cnt; c0 += MOE_MT) {
        const int mine = s_list[min(c0 + g, cnt - 1)];
        float acc[4];
        rows16_times_tokens8(lo, hi, act + (size_t)mine * F, F, c, acc);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int at = c0 + 2 * c + q;
            if (at >= cnt) continue;
            const size_t pair = s_list[at];
            if (col_lo < d) y[pair * d + col_lo] = acc[q];
            if (col_hi < d) y[pair * d + col_hi] = acc[2 + q];
        }
    }
}

static bool expert_kernels_fit(int n, int k) { return n <= MOE_LIST && (k & 7) == 0; }

RLLM_API int rllm_moe_expert_gate_up(const void* h, const void* w_gu, const int* idx, void* act, int n, int top_k, int E,
                                     int d, int F, float limit, float alpha, float shift, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || F <= 0 || top_k <= 0 || E <= 0 || !expert_kernels_fit(n, d) || ((uintptr_t)h & 15) || ((uintptr_t)w_gu & 15))
        return (int)cudaErrorInvalidValue;
    const GluForm glu = {limit, alpha, shift};
    return rllm_launch(moe_expert_gate_up_kernel, dim3(E, (F + MOE_COLS - 1) / MOE_COLS), dim3(128), 0, stream,
                       (const bf16*)h, (const bf16*)w_gu, idx, (bf16*)act, n * top_k, top_k, d, F, glu);
}

RLLM_API int rllm_moe_expert_down(const void* act, const void* w_down, const int* idx, float* y, int n, int top_k, int E,
                                  int d, int F, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || F <= 0 || top_k <= 0 || E <= 0 || !expert_kernels_fit(n, F) || ((uintptr_t)act & 15) ||
        ((uintptr_t)w_down & 15))
        return (int)cudaErrorInvalidValue;
    return rllm_launch(moe_expert_down_kernel, dim3(E, (d + MOE_DOWN_COLS - 1) / MOE_DOWN_COLS), dim3(128), 0, stream,
                       (const bf16*)act, (const bf16*)w_down, idx, y, n * top_k, d, F);
}

// ------------------------------------------------------------------ many rows: pairs in expert order
// counts[e], offsets[e] (E + 1 entries) and place[pair]: the pair's row among all pairs sorted by expert,
// pairs of one expert in pair order (stable), so the order never depends on scheduling.  A block takes 32
// experts, a warp one: every block counts all pairs (shared-memory atomics; integer sums have no order),
// then a warp walks the pairs 32 at a time and ranks its expert's pairs by a ballot.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ idx, int n_pairs, int E, int* offsets, int* place) {
    __shared__ int s_count[MOE_MAX_EXPERTS + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int e = tid; e <= E; e += blockDim.x) s_count[e] = 0;
    __syncthreads();
    for (int p = tid; p < n_pairs; p += blockDim.x) atomicAdd(&s_count[idx[p]], 1);
    __syncthreads();
    if (warp == 0) {                                       // exclusive prefix sum over the experts, 32 at a time
        int run = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane, c = e < E ? s_count[e] : 0;
            int incl = c;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, m);
                if (lane >= m) incl += up;
            }
            if (e < E) s_count[e] = run + incl - c;
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_count[E] = run;
    }
    __syncthreads();
    if (blockIdx.x == 0)
        for (int e = tid; e <= E; e += blockDim.x) offsets[e] = s_count[e];
    const int e = blockIdx.x * 32 + warp;
    if (e >= E || s_count[e + 1] == s_count[e]) return;
    int at = s_count[e];
    for (int p0 = 0; p0 < n_pairs; p0 += 32) {
        const int p = p0 + lane;
        const bool mine = p < n_pairs && idx[p] == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) place[p] = at + __popc(m & ((1u << lane) - 1u));
        at += __popc(m);
    }
}

RLLM_API int rllm_moe_sort(const int* idx, int n_pairs, int E, int* offsets, int* place, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || E > MOE_MAX_EXPERTS) return (int)cudaErrorInvalidValue;
    return rllm_launch(moe_sort_kernel, dim3((E + 31) / 32), dim3(1024), 0, stream, idx, n_pairs, E, offsets, place);
}

// rows[place[pair]] = h[pair / top_k]: a block per token reads the row once (16 bytes a thread and turn where the
// rows allow it) and writes it to the places of its top_k pairs
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const T* h, const int* __restrict__ place, T* rows, int top_k, int d, int vec) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const T* src = h + (size_t)t * d;
    if (vec) {
        const int n16 = (int)((size_t)d * sizeof(T) / 16);
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) {
            const uint4 u = s4[i];
            for (int j = 0; j < top_k; ++j)
                reinterpret_cast<uint4*>(rows + (size_t)place[(size_t)t * top_k + j] * d)[i] = u;
        }
        return;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const T v = src[i];
        for (int j = 0; j < top_k; ++j) rows[(size_t)place[(size_t)t * top_k + j] * d + i] = v;
    }
}

RLLM_API int rllm_moe_gather_rows(const void* h, int dt, const int* place, void* rows, int n_pairs, int top_k, int d,
                                  cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (top_k <= 0 || n_pairs % top_k) return (int)cudaErrorInvalidValue;
    const size_t row_bytes = (size_t)d * (dt == RLLM_F32 ? 4 : 2);
    const int vec = row_bytes % 16 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)rows & 15) == 0;
    const dim3 grid(n_pairs / top_k), block(row_bytes >= 4096 ? 256 : 128);
    if (dt == RLLM_F32)
        return rllm_launch(moe_gather_rows_kernel<float>, grid, block, 0, stream, (const float*)h, place, (float*)rows,
                           top_k, d, vec);
    return rllm_launch(moe_gather_rows_kernel<bf16>, grid, block, 0, stream, (const bf16*)h, place, (bf16*)rows, top_k, d,
                       vec);
}

// out[t] = sum_j weight[t, j] * y[place[t * top_k + j]] (+ shared[t] * sigmoid(gate[t])); place null: y in pair order
// A thread takes four neighbouring columns where the rows allow it (16-byte loads, a token's top_k rows in flight
// side by side), one column otherwise; the columns of a token are spread over blockIdx.y.
template <int VEC>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* y, const int* place, const float* weight, float* out, const float* shared,
                   const float* gate, long long ld_gate, int top_k, int d) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
    if (i >= d) return;
    const float sg = (shared && gate) ? 1.0f / (1.0f + expf(-gate[(size_t)t * ld_gate])) : 1.0f;
    float sum[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) sum[v] = 0.f;
#pragma unroll 4
    for (int j = 0; j < top_k; ++j) {
        const float w = weight[(size_t)t * top_k + j];
        const float* row = y + (size_t)(place ? place[(size_t)t * top_k + j] : t * top_k + j) * d + i;
        if constexpr (VEC == 4) {
            const float4 r = *reinterpret_cast<const float4*>(row);
            sum[0] += w * r.x;
            sum[1] += w * r.y;
            sum[2] += w * r.z;
            sum[3] += w * r.w;
        } else {
            sum[0] += w * row[0];
        }
    }
    if constexpr (VEC == 4) {
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (shared) s4 = *reinterpret_cast<const float4*>(shared + (size_t)t * d + i);
        *reinterpret_cast<float4*>(out + (size_t)t * d + i) =
            make_float4(sum[0] + s4.x * sg, sum[1] + s4.y * sg, sum[2] + s4.z * sg, sum[3] + s4.w * sg);
    } else {
        out[(size_t)t * d + i] = sum[0] + (shared ? shared[(size_t)t * d + i] * sg : 0.f);
    }
}

RLLM_API int rllm_moe_combine(const float* y, const int* place, const float* weight, float* out, const float* shared,
                              const float* gate, long long ld_gate, int n, int top_k, int d, cudaStream_t stream) {
    if (n <= 0) return 0;
    const auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if ((d & 3) == 0 && al16(y) && al16(out) && al16(shared)) {
        const int threads = d >= 1024 ? 256 : 128;
        return rllm_launch(moe_combine_kernel<4>, dim3(n, (d / 4 + threads - 1) / threads), dim3(threads), 0, stream, y,
                           place, weight, out, shared, gate, ld_gate, top_k, d);
    }
    const int threads = d >= 256 ? 256 : 128;
    return rllm_launch(moe_combine_kernel<1>, dim3(n, (d + threads - 1) / threads), dim3(threads), 0, stream, y, place,
                       weight, out, shared, gate, ld_gate, top_k, d);
}

RLLM_PACKED(rllm_moe_route)
RLLM_PACKED(rllm_moe_pairs_gate_up)
RLLM_PACKED(rllm_moe_pairs_down)
RLLM_PACKED(rllm_moe_expert_gate_up)
RLLM_PACKED(rllm_moe_expert_down)
RLLM_PACKED(rllm_moe_sort)
RLLM_PACKED(rllm_moe_gather_rows)
RLLM_PACKED(rllm_moe_combine)
