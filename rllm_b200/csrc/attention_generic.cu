// Paged causal attention, plain form: one block per (token, query head), float32
// arithmetic, any head size up to 512 (keys: 2048), any page size, any
// number of heads and groups, optional sliding window.  It is the float32 path of
// the engine and the reference the tensor-core kernels are tested against.
//
// Token t of request r = seq_ids[t] at absolute position pos sees keys p with
// max(0, pos+1-window) <= p <= pos (window 0: all keys) and, with keep_first > 0, also the
// keys p < keep_first that the window has left behind (they keep their positions; a model
// without position encoding in the scores sees no difference).  The keys of the step's own
// tokens are already in the cache.  Key p lives in page block_table[r][p / bs] at
// offset p % bs; cache layouts [page][kv_head][bs][hd] for keys and [page][kv_head][bs][hdv]
// for values (the value heads may have another size; the output is [n, H * hdv]).  Value rows lie
// v_ld elements apart (hdv when they have a pool of their own; the key rows' length when the values
// are the leading entries of the key rows themselves, v_cache == k_cache).
// chunk > 0: positions are cut into runs of `chunk` counted from 0 and a token sees only the keys of
// its own run (p >= pos - pos % chunk).  softcap > 0: a score s becomes softcap * tanh(s / softcap)
// before the softmax.  sink (one number per query head, or null): the softmax's denominator also holds
// exp(sink[h]), which stands for no key and adds no value.
//
// Formula: crates/rllm-cpu/src/lib.rs:389-425 of AxiomOperator/rllm; its device
// counterpart is paged_attention (crates/rllm-cuda/kernels/kernels.cu:1634-1690).
// Keys are consumed in chunks of 128 in ascending order with an online softmax, so
// the result for a token depends only on its own keys, never on the batch around it.
#include "common.cuh"
#include <math.h>

#define ATT_THREADS 128
#define ATT_MAX_ACC 4   // value heads: hdv <= ATT_THREADS * ATT_MAX_ACC (key heads up to 2048)

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const TQ* q, const TC* k_cache,
                               const TC* v_cache, TO* out,
                               const int* __restrict__ positions, const int* __restrict__ seq_ids,
                               const int* __restrict__ block_table, int table_stride, int H, int K,
                               int hd, int hdv, int bs, float scale, int window, int keep_first, int n_pages,
                               int* err, int chunk, float softcap, int v_ld, const float* __restrict__ sink) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_launch_dependents();
    float* qs = smem;                    // [hd]
    float* pr = smem + hd;               // [ATT_THREADS] probabilities of the chunk
    int* rowoff = (int*)(pr + ATT_THREADS);  // [ATT_THREADS] element offset / hd of each key row
    __shared__ float red[33];

    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (H / K);
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_ids[t] * table_stride;
    int first = (window > 0 && pos + 1 - window > 0) ? pos + 1 - window : 0;
    if (chunk > 0) first = max(first, pos - pos % chunk);
    const int tid = threadIdx.x;

    const TQ* qrow = q + ((size_t)t * H + h) * hd;
    for (int i = tid; i < hd; i += ATT_THREADS) qs[i] = to_f<TQ>(qrow[i]);
    __syncthreads();

    float acc[ATT_MAX_ACC];
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) acc[a] = 0.f;
    // a sink: a term exp(sink[h]) in the denominator that has no key and no value
    float m_run = sink ? sink[h] : -INFINITY, l_run = sink ? 1.f : 0.f;

    // two runs of keys: the kept first ones outside the window, then the window
    const int kept = keep_first < first ? keep_first : first;
    for (int run = 0; run < 2; ++run) {
    const int lo = run == 0 ? 0 : first, hi = run == 0 ? kept : pos + 1;
    for (int c0 = lo; c0 < hi; c0 += ATT_THREADS) {
        const int p = c0 + tid;
        float s = -INFINITY;
        if (p < hi) {
            int page = table[p / bs];
            if (page < 0 || page >= n_pages) {        // refused: read page 0, report
                if (err) atomicExch(err, RLLM_ERR_PAGE);
                page = 0;
            }
            const size_t row = ((size_t)page * K + kvh) * bs + (p % bs);
            rowoff[tid] = (int)row;
            const TC* kr = k_cache + row * hd;
            float dot = 0.f;
            for (int i = 0; i < hd; ++i) dot += qs[i] * to_f<TC>(kr[i]);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        }
        const float cmax = block_max(s, red);
        const float m_new = fmaxf(m_run, cmax);
        const float e = (p < hi) ? expf(s - m_new) : 0.f;
        pr[tid] = e;
        const float csum = block_sum(e, red);          // also orders pr/rowoff writes before reads
        const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * alpha + csum;
        m_run = m_new;
        const int cn = min(ATT_THREADS, hi - c0);
#pragma unroll
        for (int a = 0; a < ATT_MAX_ACC; ++a) {
            const int d = tid + a * ATT_THREADS;
            if (d < hdv) {
                float v = acc[a] * alpha;
                for (int j = 0; j < cn; ++j) v += pr[j] * to_f<TC>(v_cache[(size_t)rowoff[j] * v_ld + d]);
                acc[a] = v;
            }
        }
        __syncthreads();
    }
    }
    TO* orow = out + ((size_t)t * H + h) * hdv;
    const float inv = 1.0f / l_run;
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) {
        const int d = tid + a * ATT_THREADS;
        if (d < hdv) orow[d] = from_f<TO>(acc[a] * inv);
    }
}

RLLM_API int rllm_paged_attention_generic(const void* q, int q_dtype, const void* k_cache,
                                          const void* v_cache, int cache_dtype, void* out,
                                          int out_dtype, const int* positions, const int* seq_ids,
                                          const int* block_table, int table_stride, int n, int H,
                                          int K, int hd, int hdv, int bs, float scale, int window, int keep_first,
                                          int n_pages, int* err, int chunk, float softcap, int v_ld,
                                          const float* sink, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (v_ld <= 0) v_ld = hdv;
    if (chunk < 0 || v_ld < hdv) return (int)cudaErrorInvalidValue;
    if (hd > 2048 || hdv > ATT_THREADS * ATT_MAX_ACC || hdv <= 0 || K <= 0 || H % K != 0 ||
        bs <= 0 || keep_first < 0)
        return (int)cudaErrorInvalidValue;
    if (q_dtype != cache_dtype || q_dtype != out_dtype) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(hd + 2 * ATT_THREADS) * sizeof(float);
    dim3 grid(n, H);
    if (q_dtype == RLLM_F32)
        return rllm_launch(paged_attention_generic_kernel<float, float, float>, grid, dim3(ATT_THREADS), smem,
                           stream, (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out,
                           positions, seq_ids, block_table, table_stride, H, K, hd, hdv, bs, scale, window, keep_first, n_pages,
                           err, chunk, softcap, v_ld, sink);
    return rllm_launch(paged_attention_generic_kernel<bf16, bf16, bf16>, grid, dim3(ATT_THREADS), smem, stream,
                       (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions,
                       seq_ids, block_table, table_stride, H, K, hd, hdv, bs, scale, window, keep_first, n_pages, err,
                       chunk, softcap, v_ld, sink);
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_paged_attention_generic)
