// Row-wise helpers that several kinds of layers share; float32 arithmetic whatever the storage
// type, accurate expf / tanhf / log1pf (no fast-math):
//
//   rows_act        out[t, c] = f1(in[t, c] + bias[c]) * f2(mul[t, c / mul_group])   (bias, mul optional;
//                   mul_group > 1: one factor for each run of that many columns, a gate per head)
//   axpby           out = a * x + b * y                                      (float32)
//   cat2_cast       out[t] = [x[t] + s * delta[t] | y[t]] in the activation type (delta optional)
//   qkv_rownorm_store  biased q/k/v projection row -> RMSNorm over the WHOLE q row and the whole k
//                   row (one weight per column), then optionally the rotation of the first `rot` entries
//                   of every query and key head by the step's angles; queries out, keys and values into
//                   the paged cache; the value heads may have another size than the key heads
//
// f1, f2: 0 identity, 1 silu z / (1 + e^-z), 2 relu(z)^2, 3 sigmoid, 4 tanh, 5 softplus.
#include "common.cuh"
#include <math.h>

enum : int { ACT_NONE = 0, ACT_SILU = 1, ACT_RELU2 = 2, ACT_SIGMOID = 3, ACT_TANH = 4, ACT_SOFTPLUS = 5 };

__device__ __forceinline__ float act_apply(float z, int act) {
    switch (act) {
        case ACT_SILU: return z / (1.0f + expf(-z));
        case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
        case ACT_SIGMOID: return 1.0f / (1.0f + expf(-z));
        case ACT_TANH: return tanhf(z);
        case ACT_SOFTPLUS: return z > 20.f ? z : log1pf(expf(z));
        default: return z;
    }
}
__device__ __forceinline__ float ld_any(const void* p, int dt, size_t i) {
    return dt == RLLM_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int dt, size_t i, float v) {
    if (dt == RLLM_F32) ((float*)p)[i] = v;
    else ((bf16*)p)[i] = __float2bfloat16_rn(v);
}

__global__ void rows_act_kernel(const void* in, int in_dt, long long in_stride, const float* __restrict__ bias,
                                int act1, const void* mul, int mul_dt, long long mul_stride, int act2, void* out,
                                int out_dt, long long out_stride, int cols, size_t total, int mul_group) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    float v = ld_any(in, in_dt, t * in_stride + c);
    if (bias) v += bias[c];
    v = act_apply(v, act1);
    if (mul) v *= act_apply(ld_any(mul, mul_dt, t * mul_stride + c / mul_group), act2);
    st_any(out, out_dt, t * out_stride + c, v);
}

// The gate of an attention's heads on bfloat16 rows: out[t, c] = in[t, c] * f2(mul[t, c / group]) with eight
// columns (16 bytes) a thread; `group` a multiple of 8, so the eight share a factor.
__global__ void rows_gate_bf16_kernel(const bf16* in, long long in_stride, const float* mul, long long mul_stride, int act2,
                                      bf16* out, long long out_stride, int cols8, int group8, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols8;
    const int c8 = (int)(i - t * cols8);
    const float f = act_apply(mul[t * mul_stride + c8 / group8], act2);
    uint4 u = *reinterpret_cast<const uint4*>(in + t * in_stride + 8 * (size_t)c8);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 v = __bfloat1622float2(p[q]);
        p[q] = __floats2bfloat162_rn(v.x * f, v.y * f);
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + 8 * (size_t)c8) = u;
}

RLLM_API int rllm_rows_act(const void* in, int in_dt, long long in_stride, const float* bias, int act1,
                           const void* mul, int mul_dt, long long mul_stride, int act2, void* out, int out_dt,
                           long long out_stride, int n, int cols, int mul_group, cudaStream_t stream) {
    const size_t total = (size_t)n * cols;
    if (total == 0) return 0;
    if (mul_group <= 0) return (int)cudaErrorInvalidValue;
    const auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (in_dt == RLLM_BF16 && out_dt == RLLM_BF16 && mul && mul_dt == RLLM_F32 && !bias && act1 == ACT_NONE &&
        mul_group % 8 == 0 && cols % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && al16(in) && al16(out)) {
        const size_t t8 = total / 8;
        return rllm_launch(rows_gate_bf16_kernel, dim3((unsigned)((t8 + 255) / 256)), dim3(256), 0, stream, (const bf16*)in,
                           in_stride, (const float*)mul, mul_stride, act2, (bf16*)out, out_stride, cols / 8, mul_group / 8, t8);
    }
    return rllm_launch(rows_act_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, in, in_dt,
                       in_stride, bias, act1, mul, mul_dt, mul_stride, act2, out, out_dt, out_stride, cols, total,
                       mul_group);
}

__global__ void axpby_kernel(float a, const float* x, float b, const float* y, float* out, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = a * x[i] + b * y[i];
}
RLLM_API int rllm_axpby(float a, const float* x, float b, const float* y, float* out, long long total,
                        cudaStream_t stream) {
    if (total <= 0) return 0;
    return rllm_launch(axpby_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, a, x, b, y, out,
                       (size_t)total);
}

// out[t, 0:d] = x[t] (+ s * delta[t]),  out[t, d:2d] = y[t]; x and y float32 [n, d].
__global__ void cat2_cast_kernel(const float* x, const void* delta, int delta_dt, float s, const float* y, void* out,
                                 int out_dt, int d, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / d;
    const int c = (int)(i - t * d);
    float v = x[i];
    if (delta) v += s * ld_any(delta, delta_dt, i);
    st_any(out, out_dt, t * 2 * d + c, v);
    st_any(out, out_dt, t * 2 * d + d + c, y[i]);
}
RLLM_API int rllm_cat2_cast(const float* x, const void* delta, int delta_dt, float s, const float* y, void* out,
                            int out_dt, int n, int d, cudaStream_t stream) {
    const size_t total = (size_t)n * d;
    if (total == 0) return 0;
    return rllm_launch(cat2_cast_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, delta,
                       delta_dt, s, y, out, out_dt, d, total);
}

// One block per token.  qkv[t] = [q (wq) | k (wk) | v (wv) | ...] with rows `ld` apart (the projection
// may hold more columns behind v, an output gate for instance) (+ bias); q and k rows are divided by
// their root mean square over the whole row (eps inside the root) and multiplied by a weight per
// column when the weight is given; q -> q_out[t]; k, v -> the paged cache at slots[t]
// (layouts [page][kv_head][bs][dk] and [page][kv_head][bs][dv]); slot < 0 writes nothing, a slot
// beyond the pool sets the error word.
// STAGED: the q and k columns (with their bias) are read from global memory once, into shared memory
// ((wq + wk) floats), and the norm, the rotation and its partner reads work from there.
template <typename TI, typename TO, bool STAGED>
__global__ void __launch_bounds__(1024)
qkv_rownorm_store_kernel(const TI* qkv, const float* __restrict__ bias, const float* __restrict__ q_norm_w,
                         const float* __restrict__ k_norm_w, const int* __restrict__ slots, TO* q_out, TO* k_cache,
                         TO* v_cache, long long ld, int wq, int wk, int wv, int G, int dk, int dv, int bs, float eps,
                         int write_kv, int n_slots, int* err, const float2* cs_table, int rot, int pairs) {
    __shared__ float red[33];
    extern __shared__ float staged_row[];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const TI* row = qkv + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int c = tid; c < wq; c += blockDim.x) {
        const float v = to_f<TI>(row[c]) + (bias ? bias[c] : 0.f);
        if (STAGED) staged_row[c] = v;
        sq += v * v;
    }
    for (int c = tid; c < wk; c += blockDim.x) {
        const float v = to_f<TI>(row[wq + c]) + (bias ? bias[wq + c] : 0.f);
        if (STAGED) staged_row[wq + c] = v;
        sk += v * v;
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = q_norm_w ? 1.0f / sqrtf(sq / (float)wq + eps) : 1.f;
    const float rk = k_norm_w ? 1.0f / sqrtf(sk / (float)wk + eps) : 1.f;
    // The rotation: entry e of a head's first `rot` turns with its partner (e +- rot/2, or its neighbour
    // in the pair layout) by the token's angle of that pair; a thread reads both normed values.
    const int half = rot >> 1;
    const float2* cs = rot ? cs_table + (size_t)t * half : nullptr;
    auto normed = [&](int base, int c, const float* w, float r) {
        float v = STAGED ? staged_row[base + c] : to_f<TI>(row[base + c]) + (bias ? bias[base + c] : 0.f);
        if (w) v = v * r * w[c];
        return v;
    };
    auto turned = [&](int base, int c, const float* w, float r) {
        const float v = normed(base, c, w, r);
        const int e = c % dk;
        if (e >= rot) return v;
        int pair, other;
        bool first;
        if (pairs) { pair = e >> 1; first = !(e & 1); other = first ? c + 1 : c - 1; }
        else { first = e < half; pair = first ? e : e - half; other = first ? c + half : c - half; }
        const float o = normed(base, other, w, r);
        const float2 a = cs[pair];
        return first ? v * a.x - o * a.y : v * a.x + o * a.y;
    };
    for (int c = tid; c < wq; c += blockDim.x) q_out[(size_t)t * wq + c] = from_f<TO>(turned(0, c, q_norm_w, rq));
    if (!write_kv) return;
    int slot = slots[t];
    if (slot >= n_slots) {
        if (tid == 0 && err) atomicExch(err, RLLM_ERR_SLOT);
        slot = -1;
    }
    if (slot < 0) return;
    const size_t page = slot / bs, off = slot % bs;
    for (int c = tid; c < wk; c += blockDim.x)
        k_cache[((page * G + c / dk) * bs + off) * dk + c % dk] = from_f<TO>(turned(wq, c, k_norm_w, rk));
    for (int c = tid; c < wv; c += blockDim.x) {
        const float v = to_f<TI>(row[wq + wk + c]) + (bias ? bias[wq + wk + c] : 0.f);
        v_cache[((page * G + c / dv) * bs + off) * dv + c % dv] = from_f<TO>(v);
    }
}

RLLM_API int rllm_qkv_rownorm_store(const void* qkv, int in_dt, long long ld, const float* bias, const float* q_norm_w,
                                    const float* k_norm_w, const int* slots, void* q_out, void* k_cache,
                                    void* v_cache, int out_dt, int n, int H, int G, int dk, int dv, int bs,
                                    float eps, int write_kv, long long n_slots, int* err, const void* cs_table,
                                    int rot, int pairs, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || bs <= 0 || ld < (long long)H * dk + (long long)G * (dk + dv) ||
        rot < 0 || rot > dk || (rot & 1) || (rot && !cs_table))
        return (int)cudaErrorInvalidValue;
    const int ns = (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots);
    // a block per token: few tokens (a decode step) get more threads each, since the row's sums keep it in one block
    const int threads = n < 128 ? 1024 : 256;
    const size_t smem = (size_t)(H + G) * dk * sizeof(float);
#define LAUNCH(TI, TO)                                                                                         \
    if (smem <= 40 * 1024)                                                                                     \
        return rllm_launch(qkv_rownorm_store_kernel<TI, TO, true>, dim3(n), dim3(threads), smem, stream, (const TI*)qkv, \
                           bias, q_norm_w, k_norm_w, slots, (TO*)q_out, (TO*)k_cache, (TO*)v_cache, ld, H * dk, G * dk, \
                           G * dv, G, dk, dv, bs, eps, write_kv, ns, err, (const float2*)cs_table, rot, pairs);    \
    return rllm_launch(qkv_rownorm_store_kernel<TI, TO, false>, dim3(n), dim3(threads), 0, stream, (const TI*)qkv, bias, \
                       q_norm_w, k_norm_w, slots, (TO*)q_out, (TO*)k_cache, (TO*)v_cache, ld, H * dk, G * dk, G * dv, \
                       G, dk, dv, bs, eps, write_kv, ns, err, (const float2*)cs_table, rot, pairs)
    if (in_dt == RLLM_F32 && out_dt == RLLM_F32) { LAUNCH(float, float); }
    if (in_dt == RLLM_F32 && out_dt == RLLM_BF16) { LAUNCH(float, bf16); }
    if (in_dt == RLLM_BF16 && out_dt == RLLM_BF16) { LAUNCH(bf16, bf16); }
    return (int)cudaErrorInvalidValue;
#undef LAUNCH
}

RLLM_PACKED(rllm_rows_act)
RLLM_PACKED(rllm_axpby)
RLLM_PACKED(rllm_cat2_cast)
RLLM_PACKED(rllm_qkv_rownorm_store)
