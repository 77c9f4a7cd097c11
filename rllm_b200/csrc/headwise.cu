// Kernels of layers that norm a sublayer's OUTPUT, of attention whose queries and keys are rotated
// first and normed afterwards, and of attention through low-rank latents.  float32 arithmetic
// whatever the storage type; accurate expf / tanhf / sqrtf (no fast-math).
//
//   norm_rows          v = in[t] / rms(in[t]) * w  (+ x[t]);  x[t] = v (float32, optional);
//                      low[t] = v in the activation type (optional).  The embedding's norm, the norm
//                      of a sublayer's output joining the stream, the norm of a latent.
//   rope_unitnorm_store  per head of a [q | k] projection row: rotate the first `rot` entries by the
//                      step's angles (pairs (i, i + rot/2)), then divide the head by its root mean
//                      square; queries out, keys into the paged cache; the values written beside them
//                      are the key heads as projected (before rotation and norm), or the columns that
//                      follow the keys when the row has them.
//   latent_rope_store  one cache row per token [normed latent (rank) | rotated shared key part (r)],
//                      and the rotated part of every query head copied behind that head's latent-space
//                      query.
//   head_norm_rope_store  per head of a [q | k | v] projection row: RMS norm with a weight, then the
//                      rotation of the first `rot` entries (either pair layout); queries out, keys and
//                      values (heads of another size) into the paged cache; rows of queries only too.
//   join_norm_rows     x += y / rms(y) * w_out and out = x / rms(x) * w_next in one pass: a norm on a
//                      sublayer's output followed by the norm in front of the next sublayer.
//   sum_norm_rows      x = (alpha * x + y) / rms(alpha * x + y) * w: the norm stands AFTER the residual sum
//                      and the normed rows ARE the stream; low[t] = x in the activation type (optional).
//   glu_clamped        out = g * sigmoid(alpha * g) * (u + shift), g = min(gate, limit),
//                      u = clamp(up, -limit, limit); alpha 0: the tanh form of gelu in place of
//                      g * sigmoid(alpha * g).
//   softcap_rows       x = cap * tanh(x / cap) in place.
//   masked_softmax_rows  a portion's score rows against its request's keys -> probabilities (causal,
//                      optionally chunked and capped), for attention written as two library products.
//
// Angles come from a table of (cos, sin) per token and pair (rope_table: once per pass).  A slot < 0
// writes nothing to the cache; a slot beyond the pool sets the error word.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float ld_dt(const void* p, int dt, size_t i) {
    return dt == RLLM_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}
__device__ __forceinline__ void st_dt(void* p, int dt, size_t i, float v) {
    if (dt == RLLM_F32) ((float*)p)[i] = v;
    else ((bf16*)p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------ norm of rows, joined to the stream
// One block per row.  `in` may be x itself (add == 0: x is normed in place).
__global__ void __launch_bounds__(256)
norm_rows_kernel(const void* in, int in_dt, long long ld_in, const float* __restrict__ w, float* x, int add,
                 void* low, int low_dt, long long ld_low, int d, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = ld_dt(in, in_dt, t * ld_in + i);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = ld_dt(in, in_dt, t * ld_in + i) * rs * (w ? w[i] : 1.f);
        if (x) {
            if (add) v += x[t * d + i];
            x[t * d + i] = v;
        }
        if (low) st_dt(low, low_dt, t * ld_low + i, v);
    }
}

// The same for float32 input whose rows, weight and outputs allow 16-byte accesses (d and the row strides
// multiples of 4): four columns a thread and pass.  The sums are taken in another order than in the kernel
// above; which of the two runs depends on the sizes and addresses only, never on the batch.
template <typename TL>
__global__ void __launch_bounds__(1024)
norm_rows_vec_kernel(const float* in, long long ld_in, const float* __restrict__ w, float* x, int add, TL* low,
                     long long ld_low, int d, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const float* row = in + t * ld_in;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(row + i);
        const float4 ww = w ? *reinterpret_cast<const float4*>(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        v.x *= rs * ww.x; v.y *= rs * ww.y; v.z *= rs * ww.z; v.w *= rs * ww.w;
        if (x) {
            float4* xp = reinterpret_cast<float4*>(x + t * d + i);
            if (add) {
                const float4 o = *xp;
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            *xp = v;
        }
        if (low) {
            TL* lp = low + t * ld_low + i;
            if (sizeof(TL) == 4) {
                *reinterpret_cast<float4*>(lp) = v;
            } else {
                __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
                uint2 u;
                u.x = *reinterpret_cast<uint32_t*>(&a);
                u.y = *reinterpret_cast<uint32_t*>(&b);
                *reinterpret_cast<uint2*>(lp) = u;
            }
        }
    }
}

RLLM_API int rllm_norm_rows(const void* in, int in_dt, long long ld_in, const float* w, float* x, int add, void* low,
                            int low_dt, long long ld_low, int n, int d, float eps, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || ld_in < d || (low && ld_low < d)) return (int)cudaErrorInvalidValue;
    const bool vec = in_dt == RLLM_F32 && d % 4 == 0 && ld_in % 4 == 0 && ((uintptr_t)in & 15) == 0 &&
                     ((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0 &&
                     (!low || (ld_low % 4 == 0 && ((uintptr_t)low & (low_dt == RLLM_F32 ? 15 : 7)) == 0));
    if (vec) {
        // few rows (a decode step): more threads a row, since the row's sum keeps it in one block
        int threads = n < 128 ? 1024 : 256;
        while (threads > 32 && threads * 4 > d) threads >>= 1;
        if (low_dt == RLLM_F32)
            return rllm_launch(norm_rows_vec_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)in, ld_in, w,
                               x, add, (float*)low, ld_low, d, eps);
        return rllm_launch(norm_rows_vec_kernel<bf16>, dim3(n), dim3(threads), 0, stream, (const float*)in, ld_in, w, x,
                           add, (bf16*)low, ld_low, d, eps);
    }
    return rllm_launch(norm_rows_kernel, dim3(n), dim3(d >= 1024 ? 256 : 128), 0, stream, in, in_dt, ld_in, w, x, add,
                       low, low_dt, ld_low, d, eps);
}

// ------------------------------------------------------------------ rotate, then unit norm, then store
// Grid (token, group of 4 heads), one warp per head; heads 0..H-1 are queries, H..H+G-1 keys.
// row = [q (H*hd) | k (G*hd) | v (G*hd, only when v_tied == 0)], rows ld apart.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
rope_unitnorm_store_kernel(const TI* row_base, long long ld, const float2* cs_table, int rot, float cs_mult,
                           const int* __restrict__ slots, TO* q_out, TO* k_cache, TO* v_cache, int H, int G, int hd,
                           int bs, float eps, int unit_norm, int v_tied, int write_kv, int n_slots, int* err) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * 4 + warp;
    if (head >= H + G) return;
    float* v = sm + (size_t)warp * hd;
    const TI* src = row_base + (size_t)t * ld + (size_t)head * hd;
    for (int i = lane; i < hd; i += 32) v[i] = to_f<TI>(src[i]);
    __syncwarp();
    const bool is_key = head >= H;
    int slot = -1;
    if (is_key && write_kv) {
        slot = slots[t];
        if (slot >= n_slots) {
            if (lane == 0 && err) atomicExch(err, RLLM_ERR_SLOT);
            slot = -1;
        }
    }
    const size_t cache_row = slot < 0 ? 0 : (((size_t)(slot / bs) * G + (head - H)) * bs + slot % bs) * hd;
    if (is_key && slot >= 0) {
        // the values: the key head as projected, or the row's own value columns
        const TI* vs = v_tied ? src : src + (size_t)G * hd;
        for (int i = lane; i < hd; i += 32) v_cache[cache_row + i] = from_f<TO>(to_f<TI>(vs[i]));
    }
    const int half = rot >> 1;
    const float2* cs = cs_table + (size_t)t * half;
    for (int i = lane; i < half; i += 32) {
        const float2 a = cs[i];
        const float c = a.x * cs_mult, s = a.y * cs_mult;
        const float u = v[i], w = v[i + half];
        v[i] = u * c - w * s;
        v[i + half] = w * c + u * s;
    }
    __syncwarp();
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) ss += v[i] * v[i];
    ss = warp_sum(ss);
    const float rs = unit_norm ? 1.0f / sqrtf(ss / (float)hd + eps) : 1.f;
    if (!is_key) {
        TO* dst = q_out + ((size_t)t * H + head) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TO>(v[i] * rs);
    } else if (slot >= 0) {
        for (int i = lane; i < hd; i += 32) k_cache[cache_row + i] = from_f<TO>(v[i] * rs);
    }
}

RLLM_API int rllm_rope_unitnorm_store(const void* rows, int in_dt, long long ld, const void* cs_table, int rot,
                                      float cs_mult, const int* slots, void* q_out, void* k_cache, void* v_cache,
                                      int out_dt, int n, int H, int G, int hd, int bs, float eps, int unit_norm,
                                      int v_tied, int write_kv, long long n_slots, int* err, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || G <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || bs <= 0 || (rot && !cs_table) ||
        ld < (long long)(H + G * (v_tied ? 1 : 2)) * hd)
        return (int)cudaErrorInvalidValue;
    const int ns = (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots);
    const dim3 grid(n, (H + G + 3) / 4);
    const size_t smem = (size_t)4 * hd * sizeof(float);
#define LAUNCH(TI, TO)                                                                                          \
    return rllm_launch(rope_unitnorm_store_kernel<TI, TO>, grid, dim3(128), smem, stream, (const TI*)rows, ld,   \
                       (const float2*)cs_table, rot, cs_mult, slots, (TO*)q_out, (TO*)k_cache, (TO*)v_cache, H, G, \
                       hd, bs, eps, unit_norm, v_tied, write_kv, ns, err)
    if (in_dt == RLLM_F32 && out_dt == RLLM_F32) { LAUNCH(float, float); }
    if (in_dt == RLLM_F32 && out_dt == RLLM_BF16) { LAUNCH(float, bf16); }
    if (in_dt == RLLM_BF16 && out_dt == RLLM_BF16) { LAUNCH(bf16, bf16); }
    return (int)cudaErrorInvalidValue;
#undef LAUNCH
}

// ------------------------------------------------------------------ latent attention: cache row and query parts
// One block per token.  kv[t] = [latent (rank) | shared key part (r)] with rows ld_kv apart (float32);
// the latent is RMS-normed with a weight, the key part rotated (pairs (i, i + r/2), or (2i, 2i + 1) when
// `pairs`); both go to the
// token's cache row [rank + r] (one key/value head).  q[t] = H heads of [plain (dq) | rotated (r)]
// with rows ld_q apart; the rotated part of head h goes to q_att[t, h, rank : rank + r] (the first
// rank entries of each head are written by the product that takes the plain part into latent space).
template <typename TQ, typename TO>
__global__ void __launch_bounds__(256)
latent_rope_store_kernel(const TQ* q, long long ld_q, const float* kv, long long ld_kv,
                         const float* __restrict__ kv_norm_w, const float2* cs_table, float cs_mult,
                         const int* __restrict__ slots, TO* q_att, TO* cache, int H, int dq, int r, int rank, int bs,
                         float eps, int write_kv, int n_slots, int* err, int pairs) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int half = r >> 1, W = rank + r;
    const float2* cs = cs_table + (size_t)t * half;
    // queries: every (head, pair)
    for (int i = tid; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        const TQ* src = q + (size_t)t * ld_q + (size_t)h * (dq + r) + dq;
        const float2 a = cs[j];
        const float c = a.x * cs_mult, s = a.y * cs_mult;
        const int iu = pairs ? 2 * j : j, iv = pairs ? 2 * j + 1 : j + half;
        const float u = to_f<TQ>(src[iu]), w = to_f<TQ>(src[iv]);
        TO* dst = q_att + ((size_t)t * H + h) * W + rank;
        dst[iu] = from_f<TO>(u * c - w * s);
        dst[iv] = from_f<TO>(w * c + u * s);
    }
    const float* row = kv + (size_t)t * ld_kv;
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, red);
    if (!write_kv) return;
    int slot = slots[t];
    if (slot >= n_slots) {
        if (tid == 0 && err) atomicExch(err, RLLM_ERR_SLOT);
        slot = -1;
    }
    if (slot < 0) return;
    const float rs = 1.0f / sqrtf(ss / (float)rank + eps);
    TO* dst = cache + (size_t)slot * W;                 // one head: page * bs + offset is the row
    for (int i = tid; i < rank; i += blockDim.x) dst[i] = from_f<TO>(row[i] * rs * kv_norm_w[i]);
    for (int j = tid; j < half; j += blockDim.x) {
        const float2 a = cs[j];
        const float c = a.x * cs_mult, s = a.y * cs_mult;
        const int iu = pairs ? 2 * j : j, iv = pairs ? 2 * j + 1 : j + half;
        const float u = row[rank + iu], w = row[rank + iv];
        dst[rank + iu] = from_f<TO>(u * c - w * s);
        dst[rank + iv] = from_f<TO>(w * c + u * s);
    }
}

RLLM_API int rllm_latent_rope_store(const void* q, int q_dt, long long ld_q, const float* kv, long long ld_kv,
                                    const float* kv_norm_w, const void* cs_table, float cs_mult, const int* slots,
                                    void* q_att, void* cache, int out_dt, int n, int H, int dq, int r, int rank,
                                    int bs, float eps, int write_kv, long long n_slots, int* err, int pairs,
                                    cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || dq <= 0 || r <= 0 || (r & 1) || rank <= 0 || bs <= 0 || !cs_table || !kv_norm_w ||
        ld_q < (long long)H * (dq + r) || ld_kv < rank + r)
        return (int)cudaErrorInvalidValue;
    const int ns = (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots);
#define LAUNCH(TQ, TO)                                                                                           \
    return rllm_launch(latent_rope_store_kernel<TQ, TO>, dim3(n), dim3(256), 0, stream, (const TQ*)q, ld_q, kv,   \
                       ld_kv, kv_norm_w, (const float2*)cs_table, cs_mult, slots, (TO*)q_att, (TO*)cache, H, dq, r, \
                       rank, bs, eps, write_kv, ns, err, pairs)
    if (q_dt == RLLM_F32 && out_dt == RLLM_F32) { LAUNCH(float, float); }
    if (q_dt == RLLM_F32 && out_dt == RLLM_BF16) { LAUNCH(float, bf16); }
    if (q_dt == RLLM_BF16 && out_dt == RLLM_BF16) { LAUNCH(bf16, bf16); }
    return (int)cudaErrorInvalidValue;
#undef LAUNCH
}

// ------------------------------------------------------------------ norm after the residual sum
// One block per row: v = alpha * x[t] + y[t] (y in any type, rows ld_y apart), x[t] = v / rms(v) * w,
// low[t] = the same in the activation type.  The sums are taken in float32 and the row is read twice
// (it stays in L1/L2), so any width runs.
__global__ void __launch_bounds__(256)
sum_norm_rows_kernel(float* x, float alpha, const void* y, int y_dt, long long ld_y, const float* __restrict__ w,
                     void* low, int low_dt, long long ld_low, int d, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    float* xr = x + t * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = alpha * xr[i] + ld_dt(y, y_dt, t * ld_y + i);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = (alpha * xr[i] + ld_dt(y, y_dt, t * ld_y + i)) * rs * w[i];
        xr[i] = v;
        if (low) st_dt(low, low_dt, t * ld_low + i, v);
    }
}

// The same for float32 y whose rows, weight and outputs allow 16-byte accesses (d and the row strides multiples
// of 4): the row is read once and kept in registers, four columns a thread and pass.  Which of the two
// kernels runs depends on the sizes and addresses only, never on the batch.
template <typename TL, int NV>
__global__ void __launch_bounds__(256)
sum_norm_rows_vec_kernel(float* x, float alpha, const float* y, long long ld_y, const float* __restrict__ w, TL* low,
                         long long ld_low, int d, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int d4 = d >> 2;
    float4* x4 = reinterpret_cast<float4*>(x + t * d);
    const float4* y4 = reinterpret_cast<const float4*>(y + t * ld_y);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = k * 256 + threadIdx.x;
        if (i < d4) {
            const float4 a = x4[i], b = y4[i];
            v[k] = make_float4(alpha * a.x + b.x, alpha * a.y + b.y, alpha * a.z + b.z, alpha * a.w + b.w);
        } else {
            v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = k * 256 + threadIdx.x;
        if (i < d4) {
            const float4 g = w4[i];
            const float4 o = make_float4(v[k].x * rs * g.x, v[k].y * rs * g.y, v[k].z * rs * g.z, v[k].w * rs * g.w);
            x4[i] = o;
            if (low) {
                TL* lp = low + t * ld_low + 4 * (size_t)i;
                lp[0] = from_f<TL>(o.x); lp[1] = from_f<TL>(o.y); lp[2] = from_f<TL>(o.z); lp[3] = from_f<TL>(o.w);
            }
        }
    }
}

template <typename TL>
static int launch_sum_norm_vec(int n, int d, cudaStream_t stream, float* x, float alpha, const float* y, long long ld_y,
                               const float* w, TL* low, long long ld_low, float eps) {
#define SV(NV)                                                                                                    \
    return rllm_launch(sum_norm_rows_vec_kernel<TL, NV>, dim3(n), dim3(256), 0, stream, x, alpha, y, ld_y, w, low, \
                       ld_low, d, eps)
    const int nv = (d / 4 + 255) / 256;
    if (nv <= 1) { SV(1); }
    if (nv <= 2) { SV(2); }
    if (nv <= 4) { SV(4); }
    if (nv <= 8) { SV(8); }
    SV(16);
#undef SV
}

RLLM_API int rllm_sum_norm_rows(float* x, float alpha, const void* y, int y_dt, long long ld_y, const float* w,
                                void* low, int low_dt, long long ld_low, int n, int d, float eps,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || !x || !y || !w || ld_y < d || (low && ld_low < d)) return (int)cudaErrorInvalidValue;
    const auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (y_dt == RLLM_F32 && d >= 256 && d <= 16384 && (d & 3) == 0 && (ld_y & 3) == 0 && al16(x) && al16(y) && al16(w)) {
        if (!low || low_dt == RLLM_F32)
            return launch_sum_norm_vec<float>(n, d, stream, x, alpha, (const float*)y, ld_y, w, (float*)low, ld_low, eps);
        return launch_sum_norm_vec<bf16>(n, d, stream, x, alpha, (const float*)y, ld_y, w, (bf16*)low, ld_low, eps);
    }
    return rllm_launch(sum_norm_rows_kernel, dim3(n), dim3(d >= 1024 ? 256 : 128), 0, stream, x, alpha, y, y_dt, ld_y,
                       w, low, low_dt, ld_low, d, eps);
}

// ------------------------------------------------------------------ clamped gated activation
// gate_up[t] = [gate (F) | up (F)] with rows ld apart.
__global__ void glu_clamped_kernel(const void* gate_up, int in_dt, long long ld, void* out, int out_dt, int F,
                                   float limit, float alpha, float shift, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F;
    const int c = (int)(i - t * F);
    float g = ld_dt(gate_up, in_dt, t * ld + c), u = ld_dt(gate_up, in_dt, t * ld + F + c);
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    const float a = alpha == 0.f ? 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)))
                                 : g / (1.0f + expf(-alpha * g));
    st_dt(out, out_dt, i, a * (u + shift));
}

RLLM_API int rllm_glu_clamped(const void* gate_up, int in_dt, long long ld, void* out, int out_dt, int n, int F,
                              float limit, float alpha, float shift, cudaStream_t stream) {
    const size_t total = (size_t)n * F;
    if (total == 0) return 0;
    if (ld < 2LL * F) return (int)cudaErrorInvalidValue;
    return rllm_launch(glu_clamped_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, gate_up,
                       in_dt, ld, out, out_dt, F, limit, alpha, shift, total);
}

// ------------------------------------------------------------------ soft cap
__global__ void softcap_rows_kernel(float* x, float cap, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

RLLM_API int rllm_softcap_rows(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
    return rllm_launch(softcap_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, cap,
                       (size_t)total);
}

// ------------------------------------------------------------------ masked softmax over score rows
// Scores S [rows, ld] (float32) of one request's portion against its keys 0 .. n_keys-1: row = token *
// H + head, the token at position pos0 + token.  P [rows, ld_p] (bfloat16) = softmax over the visible
// keys j (j <= position; with chunk > 0 also j >= position - position % chunk) of s * scale, capped
// when softcap > 0; every other column up to n_cols is written as zero.  One block per row.
// STAGED: the row's visible scores are read once into shared memory (n_cols floats) and the other two passes
// run from there; rows too long for that read global memory three times.
template <bool STAGED>
__global__ void __launch_bounds__(256)
masked_softmax_rows_kernel(const float* S, long long ld, bf16* P, long long ld_p, int H, int pos0, int n_cols,
                           float scale, float softcap, int chunk, int window, int col0) {
    extern __shared__ float staged[];
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    const int pos = pos0 + (int)(row / H);
    // column j holds the key at position col0 + j
    int lo = chunk > 0 ? pos - pos % chunk : 0;
    if (window > 0) lo = max(lo, pos + 1 - window);
    lo = max(lo - col0, 0);
    const int hi = min(pos + 1 - col0, n_cols);
    const float* s = S + row * ld;
    bf16* p = P + row * ld_p;
    float mx = -INFINITY;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        float v = s[j] * scale;
        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
        if (STAGED) staged[j] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) {
        float v;
        if (STAGED) {
            v = staged[j] = expf(staged[j] - mx);
        } else {
            v = s[j] * scale;
            if (softcap > 0.f) v = softcap * tanhf(v / softcap);
            v = expf(v - mx);
        }
        sum += v;
    }
    sum = block_sum(sum, red);
    const float inv = 1.0f / sum;
    for (int j = threadIdx.x; j < n_cols; j += blockDim.x) {
        float e = 0.f;
        if (j >= lo && j < hi) {
            if (STAGED) {
                e = staged[j] * inv;
            } else {
                float v = s[j] * scale;
                if (softcap > 0.f) v = softcap * tanhf(v / softcap);
                e = expf(v - mx) * inv;
            }
        }
        p[j] = __float2bfloat16_rn(e);
    }
}

RLLM_API int rllm_masked_softmax_rows(const float* S, long long ld, void* P, long long ld_p, int rows, int H,
                                      int pos0, int n_cols, float scale, float softcap, int chunk, int window,
                                      int col0, cudaStream_t stream) {
    if (rows <= 0 || n_cols <= 0) return 0;
    if (H <= 0 || pos0 < 0 || ld < n_cols || ld_p < n_cols || chunk < 0 || window < 0 || col0 < 0)
        return (int)cudaErrorInvalidValue;
    if (n_cols <= 11264)                     // 44 KB: within the shared memory every launch may have
        return rllm_launch(masked_softmax_rows_kernel<true>, dim3(rows), dim3(256), (size_t)n_cols * sizeof(float),
                           stream, S, ld, (bf16*)P, ld_p, H, pos0, n_cols, scale, softcap, chunk, window, col0);
    return rllm_launch(masked_softmax_rows_kernel<false>, dim3(rows), dim3(256), 0, stream, S, ld, (bf16*)P, ld_p, H,
                       pos0, n_cols, scale, softcap, chunk, window, col0);
}

// ------------------------------------------------------------------ norm per head, then rotate, then store
// Grid (token, group of 4 heads), one warp per head; heads 0..H-1 are queries, H..H+G-1 keys (only
// with has_kv).  row = [q (H*hd) | k (G*hd) | v (G*hdv)], rows ld apart.  A query or key head is divided
// by its root mean square and multiplied by a weight of hd entries shared by all heads (null: no norm),
// then its first `rot` entries are rotated by the token's angles: pairs (2i, 2i + 1) when `pairs`, else
// (i, i + rot/2).  Queries go to q_out, keys and values (heads of hdv entries, as projected) into the
// pages.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
head_norm_rope_store_kernel(const TI* row_base, long long ld, const float* __restrict__ q_w,
                            const float* __restrict__ k_w, const float2* cs_table, int rot, int pairs,
                            const int* __restrict__ slots, TO* q_out, TO* k_cache, TO* v_cache, int H, int G, int hd,
                            int hdv, int bs, float eps, int has_kv, int write_kv, int n_slots, int* err) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * 4 + warp;
    if (head >= H + (has_kv ? G : 0)) return;
    float* v = sm + (size_t)warp * hd;
    const TI* src = row_base + (size_t)t * ld + (size_t)head * hd;
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const float x = to_f<TI>(src[i]);
        v[i] = x;
        ss += x * x;
    }
    ss = warp_sum(ss);
    const bool is_key = head >= H;
    const float* w = is_key ? k_w : q_w;
    if (w) {
        const float rs = 1.0f / sqrtf(ss / (float)hd + eps);
        for (int i = lane; i < hd; i += 32) v[i] = v[i] * rs * w[i];
    }
    __syncwarp();
    int slot = -1;
    if (is_key && write_kv) {
        slot = slots[t];
        if (slot >= n_slots) {
            if (lane == 0 && err) atomicExch(err, RLLM_ERR_SLOT);
            slot = -1;
        }
    }
    const int half = rot >> 1;
    const float2* cs = cs_table + (size_t)t * half;
    for (int i = lane; i < half; i += 32) {
        const float2 a = cs[i];
        const int iu = pairs ? 2 * i : i, iv = pairs ? 2 * i + 1 : i + half;
        const float u = v[iu], x = v[iv];
        v[iu] = u * a.x - x * a.y;
        v[iv] = x * a.x + u * a.y;
    }
    __syncwarp();
    if (!is_key) {
        TO* dst = q_out + ((size_t)t * H + head) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = from_f<TO>(v[i]);
    } else if (slot >= 0) {
        const int kh = head - H;
        const size_t page_row = ((size_t)(slot / bs) * G + kh) * bs + slot % bs;
        for (int i = lane; i < hd; i += 32) k_cache[page_row * hd + i] = from_f<TO>(v[i]);
        const TI* vs = row_base + (size_t)t * ld + (size_t)(H + G) * hd + (size_t)kh * hdv;
        for (int i = lane; i < hdv; i += 32) v_cache[page_row * hdv + i] = from_f<TO>(to_f<TI>(vs[i]));
    }
}

RLLM_API int rllm_head_norm_rope_store(const void* rows, int in_dt, long long ld, const float* q_w, const float* k_w,
                                       const void* cs_table, int rot, int pairs, const int* slots, void* q_out,
                                       void* k_cache, void* v_cache, int out_dt, int n, int H, int G, int hd, int hdv,
                                       int bs, float eps, int has_kv, int write_kv, long long n_slots, int* err,
                                       cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || G <= 0 || hd <= 0 || hdv <= 0 || rot < 0 || rot > hd || (rot & 1) || bs <= 0 || (rot && !cs_table) ||
        ld < (long long)H * hd + (has_kv ? (long long)G * (hd + hdv) : 0))
        return (int)cudaErrorInvalidValue;
    const int ns = (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots);
    const dim3 grid(n, (H + (has_kv ? G : 0) + 3) / 4);
    const size_t smem = (size_t)4 * hd * sizeof(float);
#define LAUNCH(TI, TO)                                                                                           \
    return rllm_launch(head_norm_rope_store_kernel<TI, TO>, grid, dim3(128), smem, stream, (const TI*)rows, ld,   \
                       q_w, k_w, (const float2*)cs_table, rot, pairs, slots, (TO*)q_out, (TO*)k_cache,            \
                       (TO*)v_cache, H, G, hd, hdv, bs, eps, has_kv, write_kv, ns, err)
    if (in_dt == RLLM_F32 && out_dt == RLLM_F32) { LAUNCH(float, float); }
    if (in_dt == RLLM_F32 && out_dt == RLLM_BF16) { LAUNCH(float, bf16); }
    if (in_dt == RLLM_BF16 && out_dt == RLLM_BF16) { LAUNCH(bf16, bf16); }
    return (int)cudaErrorInvalidValue;
#undef LAUNCH
}

// ------------------------------------------------------------------ a norm on an output, joined, and the next norm
// One block per row: x[t] += y[t] / rms(y[t]) * w_out, then out[t] = x[t] / rms(x[t]) * w_next in the
// activation type.  The new row of x stays in shared memory between the two halves.
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
join_norm_rows_kernel(const TY* y, long long ld_y, const float* __restrict__ w_out, float eps_out, float* x,
                      const float* __restrict__ w_next, float eps_next, TO* out, int d) {
    extern __shared__ float row[];
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = to_f<TY>(y[t * ld_y + i]);
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps_out);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = x[t * d + i] + row[i] * rs * w_out[i];
        x[t * d + i] = v;
        row[i] = v;
        s2 += v * v;
    }
    s2 = block_sum(s2, red);
    const float r2 = 1.0f / sqrtf(s2 / (float)d + eps_next);
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[t * d + i] = from_f<TO>(row[i] * r2 * w_next[i]);
}

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = u;
}

// The same with rows in registers: float32 y, d a multiple of 4 up to NV * 4 * 256, rows 16-byte aligned.
// A thread holds NV float4 of the row; all its loads are in flight at once.
template <typename TO, int NV>
__global__ void __launch_bounds__(256)
join_norm_rows_vec_kernel(const float* y, long long ld_y, const float* __restrict__ w_out, float eps_out, float* x,
                          const float* __restrict__ w_next, float eps_next, TO* out, int d) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int d4 = d >> 2;
    const float4* y4 = reinterpret_cast<const float4*>(y + t * ld_y);
    float4* x4 = reinterpret_cast<float4*>(x + t * d);
    const float4* wo4 = reinterpret_cast<const float4*>(w_out);
    const float4* wn4 = reinterpret_cast<const float4*>(w_next);
    float4 yv[NV], xv[NV];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = v * 256 + threadIdx.x;
        yv[v] = i < d4 ? y4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        xv[v] = i < d4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) ss += yv[v].x * yv[v].x + yv[v].y * yv[v].y + yv[v].z * yv[v].z + yv[v].w * yv[v].w;
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps_out);
    float s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = v * 256 + threadIdx.x;
        if (i < d4) {
            const float4 w = wo4[i];
            xv[v].x += yv[v].x * rs * w.x;
            xv[v].y += yv[v].y * rs * w.y;
            xv[v].z += yv[v].z * rs * w.z;
            xv[v].w += yv[v].w * rs * w.w;
            x4[i] = xv[v];
            s2 += xv[v].x * xv[v].x + xv[v].y * xv[v].y + xv[v].z * xv[v].z + xv[v].w * xv[v].w;
        }
    }
    s2 = block_sum(s2, red);
    const float r2 = 1.0f / sqrtf(s2 / (float)d + eps_next);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = v * 256 + threadIdx.x;
        if (i < d4) {
            const float4 w = wn4[i];
            store4(out + t * d + (size_t)i * 4, xv[v].x * r2 * w.x, xv[v].y * r2 * w.y, xv[v].z * r2 * w.z,
                   xv[v].w * r2 * w.w);
        }
    }
}

template <typename TO>
static int launch_join_norm_vec(int n, int d, cudaStream_t stream, const float* y, long long ld_y, const float* w_out,
                                float eps_out, float* x, const float* w_next, float eps_next, TO* out) {
#define JV(NV)                                                                                                     \
    return rllm_launch(join_norm_rows_vec_kernel<TO, NV>, dim3(n), dim3(256), 0, stream, y, ld_y, w_out, eps_out, x, \
                       w_next, eps_next, out, d)
    const int nv = (d / 4 + 255) / 256;
    if (nv <= 1) { JV(1); }
    if (nv <= 2) { JV(2); }
    if (nv <= 4) { JV(4); }
    if (nv <= 8) { JV(8); }
    JV(12);
#undef JV
}

RLLM_API int rllm_join_norm_rows(const void* y, int y_dt, long long ld_y, const float* w_out, float eps_out, float* x,
                                 const float* w_next, float eps_next, void* out, int out_dt, int n, int d,
                                 cudaStream_t stream) {
    if (n <= 0) return 0;
    if (d <= 0 || ld_y < d || !w_out || !w_next || !x || !out) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    const auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (y_dt == RLLM_F32 && d >= 256 && (d & 3) == 0 && (ld_y & 3) == 0 && al16(y) && al16(x) && al16(w_out) && al16(w_next) &&
        al16(out)) {
        if (out_dt == RLLM_F32)
            return launch_join_norm_vec<float>(n, d, stream, (const float*)y, ld_y, w_out, eps_out, x, w_next, eps_next, (float*)out);
        if (out_dt == RLLM_BF16)
            return launch_join_norm_vec<bf16>(n, d, stream, (const float*)y, ld_y, w_out, eps_out, x, w_next, eps_next, (bf16*)out);
    }
    const dim3 block(d >= 2048 ? 256 : 128);
#define LAUNCH(TY, TO)                                                                                          \
    return rllm_launch(join_norm_rows_kernel<TY, TO>, dim3(n), block, smem, stream, (const TY*)y, ld_y, w_out,   \
                       eps_out, x, w_next, eps_next, (TO*)out, d)
    if (y_dt == RLLM_F32 && out_dt == RLLM_F32) { LAUNCH(float, float); }
    if (y_dt == RLLM_F32 && out_dt == RLLM_BF16) { LAUNCH(float, bf16); }
    if (y_dt == RLLM_BF16 && out_dt == RLLM_BF16) { LAUNCH(bf16, bf16); }
    return (int)cudaErrorInvalidValue;
#undef LAUNCH
}

RLLM_PACKED(rllm_head_norm_rope_store)
RLLM_PACKED(rllm_join_norm_rows)
RLLM_PACKED(rllm_masked_softmax_rows)
RLLM_PACKED(rllm_norm_rows)
RLLM_PACKED(rllm_rope_unitnorm_store)
RLLM_PACKED(rllm_latent_rope_store)
RLLM_PACKED(rllm_glu_clamped)
RLLM_PACKED(rllm_sum_norm_rows)
RLLM_PACKED(rllm_softcap_rows)
