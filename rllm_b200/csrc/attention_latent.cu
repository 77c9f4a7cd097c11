// Decode-shape attention of many query heads over ONE key/value head whose values are the leading
// entries of the key rows (attention through a latent): bf16, mma.sync m16n8k16, float32 softmax.
//
// A token's H heads all read the same key rows, so they are the M side of the products: a CTA takes
// one token, 32 of its heads (two m16 tiles; grid.y walks the head chunks) and one split of SPLIT
// keys (grid.z), which it walks in tiles of 32 keys:
//
//   S[16 heads, 32 keys] = Q[16, W] . C[32 keys, W]^T        per warp: its m-tile against the whole key tile
//   softmax step over the tile, float32, in registers (a head's scores lie in the four lanes of a quad)
//   O[16 heads, V/2] += P[16, 32] . C[32 keys, half of :V]   per warp: its m-tile, one half of the value columns
//
// The two warps of an m-tile compute the same scores (the products are not the limit), so that P never
// leaves the registers and a tile costs one block barrier, for its buffer.
//
// W = key row length (latent + rotated part), V = value length (the latent).  Q and the key tile lie
// in shared memory with rows padded by 16 bytes, so that the eight 16-byte rows of every ldmatrix
// fall into eight different bank groups without a swizzle; the next key tile is on its way (cp.async,
// second buffer) while the current one is worked on.  Keys beyond the token's position are
// loaded as zeros and masked.  Every split writes its unnormalized O, max and sum; a second kernel
// merges the splits of a (token, head) in split order.  The split size is a constant, so a token's
// result does not depend on the batch around it.
//
// Needs W % 16 == 0, V % 64 == 0, V <= 512, V <= W.  Other sizes, float32 and prompt portions take
// other kernels (ops.shared_kv_attention).
#include "common.cuh"
#include <math.h>

#define LAT_HEADS 32        // heads per CTA
#define LAT_TILE 32         // keys per tile
#define LAT_PAD 8           // bf16 elements of padding per shared-memory row
#define LAT_MAX_NT 32       // n8 tiles of value columns per warp (V / 2 / 8)

__device__ __forceinline__ uint32_t lat_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lat_cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void lat_ldsm(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lat_ldsm_t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lat_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct LatentParams {
    const bf16* q;            // [n, H, W]
    const bf16* cache;        // [pages, 1, bs, W]
    float* part_o;            // [n, chunks, splits, LAT_HEADS, V]
    float* part_ml;           // [n, chunks, splits, LAT_HEADS, 2]
    const int* positions;     // [n]
    const int* seq_ids;       // [n]
    const int* block_table;   // [R, table_stride]
    int table_stride, n_pages;
    int* err;
    int H, W, V, bs, split;
    float scale, softcap;
    int window;               // > 0: a token sees only the last `window` keys (itself included)
};

__device__ __forceinline__ uint32_t lat_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(128) latent_decode_kernel(const LatentParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int LD = p.W + LAT_PAD;                                   // elements per padded row
    bf16* Qs = reinterpret_cast<bf16*>(smem);                       // [32][LD]
    bf16* Kbuf = Qs + LAT_HEADS * LD;                               // two key tiles [32][LD]: one in use, one on its way
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int tok = blockIdx.x, hc = blockIdx.y, z = blockIdx.z;
    const int head0 = hc * LAT_HEADS;
    const size_t part = ((size_t)tok * gridDim.y + hc) * gridDim.z + z;
    const int pos = p.positions[tok];
    // with a window the splits count from the window's first key rounded down to a tile, so that the
    // number of splits follows the window and not the context
    const int lo = p.window > 0 ? max(pos + 1 - p.window, 0) : 0;
    const int kb = lo / LAT_TILE * LAT_TILE + z * p.split, ke = min(pos + 1, kb + p.split);
    pdl_wait();
    if (kb >= ke) {                                                 // an empty split
        if (tid < LAT_HEADS) {
            p.part_ml[(part * LAT_HEADS + tid) * 2] = -INFINITY;
            p.part_ml[(part * LAT_HEADS + tid) * 2 + 1] = 0.f;
        }
        return;
    }
    const int* table = p.block_table + (size_t)p.seq_ids[tok] * p.table_stride;
    const int chunks = p.W / 8;                                     // 16-byte pieces of a row
    // queries of this chunk of heads; rows beyond H are zero
    // (four threads a row, each every fourth 16-byte piece: one address computation a thread)
    const int my_row = tid >> 2, my_c0 = tid & 3;
    {
        const bool live = head0 + my_row < p.H;
        const bf16* src = p.q + ((size_t)tok * p.H + (live ? head0 + my_row : 0)) * p.W;
        const uint32_t dst = lat_smem(Qs + my_row * LD);
        for (int c = my_c0; c < chunks; c += 4) lat_cp16(dst + c * 16, src + c * 8, live ? 16 : 0);
    }
    // This warp: the 16 heads of m-tile `mt` against ALL keys of a tile (so a head's scores, its softmax
    // step and its P fragments stay in this warp's registers: the two warps of an m-tile compute the same
    // scores), and for P . V the half `ch` of the value columns.
    const int mt = warp & 1, ch = warp >> 1;
    const int nt_w = p.V / 16;                                      // n8 tiles of this warp: V / 2 columns
    const int col0 = ch * (p.V / 2);
    float acc[LAT_MAX_NT][4];
#pragma unroll
    for (int j = 0; j < LAT_MAX_NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};      // rows g and g + 8; l: this lane's columns
    // ldmatrix lane addresses: A-like (rows (mi & 1) * 8 + r, columns + (mi >> 1) * 8) and B-like for the
    // keys as n (rows (mi >> 1) * 8 + r, columns + (mi & 1) * 8)
    const int mi = lane >> 3, r8 = lane & 7;
    const int a_row = (mi & 1) * 8 + r8, a_col = (mi >> 1) * 8;
    const int b_row = (mi >> 1) * 8 + r8, b_col = (mi & 1) * 8;

    // a key tile on its way: rows first .. first + 31 of the request, zeros beyond ke; one cp.async group
    auto fetch_tile = [&](bf16* dst, int first) {
        // four threads a key row: one table look-up a thread and tile, then every fourth 16-byte piece of the row
        const int key = first + my_row;
        const bool live = key < ke;
        int page = live ? table[key / p.bs] : 0;
        if ((unsigned)page >= (unsigned)p.n_pages) {
            if (p.err) atomicExch(p.err, RLLM_ERR_PAGE);
            page = 0;
        }
        const bf16* src = p.cache + ((size_t)page * p.bs + (live ? key % p.bs : 0)) * p.W;
        const uint32_t d = lat_smem(dst + my_row * LD);
        for (int c = my_c0; c < chunks; c += 4) lat_cp16(d + c * 16, src + c * 8, live ? 16 : 0);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    fetch_tile(Kbuf, kb);                                           // with the queries in the same group
    int cur = 0;
    for (int kt = kb; kt < ke; kt += LAT_TILE, cur ^= 1) {
        bf16* Ks = Kbuf + cur * LAT_TILE * LD;
        if (kt + LAT_TILE < ke) {                                   // the next tile travels while this one is worked on
            fetch_tile(Kbuf + (cur ^ 1) * LAT_TILE * LD, kt + LAT_TILE);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        // ---- S = Q K^T: 16 heads x 32 keys (four n8 tiles)
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
        {
            const uint32_t qa = lat_smem(Qs + (mt * 16 + a_row) * LD + a_col);
            const uint32_t ka = lat_smem(Ks + b_row * LD + b_col);
            const uint32_t kb16 = ka + 16 * LD * 2;                 // keys 16 .. 31
            for (int k0 = 0; k0 < p.W; k0 += 16) {
                uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                lat_ldsm(qa + k0 * 2, a0, a1, a2, a3);
                lat_ldsm(ka + k0 * 2, b0, b1, b2, b3);
                lat_mma(s[0], a0, a1, a2, a3, b0, b1);
                lat_mma(s[1], a0, a1, a2, a3, b2, b3);
                lat_ldsm(kb16 + k0 * 2, b0, b1, b2, b3);
                lat_mma(s[2], a0, a1, a2, a3, b0, b1);
                lat_mma(s[3], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- scale, cap, mask; softmax step in registers (a row's 32 scores lie in the four lanes of a quad)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * p.scale;
                if (p.softcap > 0.f) v = p.softcap * tanhf(v / p.softcap);
                const int key = kt + j * 8 + 2 * t4 + (e & 1);
                if (key >= ke || key < lo) v = -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
            mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
            const float m_new = fmaxf(m_run[x], mx[x]);                // finite: every tile of a split holds a live key
            alpha[x] = expf(m_run[x] - m_new);                         // 0 at the first tile
            m_run[x] = m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[j][e] = expf(s[j][e] - m_run[e >> 1]);               // exp(-inf) = 0
                sum[e >> 1] += s[j][e];
            }
        l_run[0] = l_run[0] * alpha[0] + sum[0];
        l_run[1] = l_run[1] * alpha[1] + sum[1];
#pragma unroll
        for (int j = 0; j < LAT_MAX_NT; ++j) {
            acc[j][0] *= alpha[0]; acc[j][1] *= alpha[0];
            acc[j][2] *= alpha[1]; acc[j][3] *= alpha[1];
        }
        // ---- O += P V over this warp's half of the value columns; P from the score registers
#pragma unroll
        for (int kk = 0; kk < LAT_TILE / 16; ++kk) {
            const uint32_t pa0 = lat_pack(s[2 * kk][0], s[2 * kk][1]), pa1 = lat_pack(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t pa2 = lat_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]), pa3 = lat_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            // V as the B operand (k = key, n = column): transposed 8x8 pieces of the key tile;
            // matrices: (keys 0-7, cols 0-7), (keys 8-15, cols 0-7), (keys 0-7, cols 8-15), (keys 8-15, cols 8-15)
            const uint32_t va = lat_smem(Ks + (kk * 16 + a_row) * LD + col0 + a_col);
#pragma unroll
            for (int jp = 0; jp < LAT_MAX_NT / 2; ++jp) {
                if (2 * jp < nt_w) {
                    uint32_t b0, b1, b2, b3;
                    lat_ldsm_t(va + jp * 32, b0, b1, b2, b3);
                    lat_mma(acc[2 * jp], pa0, pa1, pa2, pa3, b0, b1);
                    lat_mma(acc[2 * jp + 1], pa0, pa1, pa2, pa3, b2, b3);
                }
            }
        }
        __syncthreads();                                            // the tile's buffer may be written again
    }
    pdl_launch_dependents();
    // ---- this split's partial results
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        l_run[x] += __shfl_xor_sync(0xffffffffu, l_run[x], 1);
        l_run[x] += __shfl_xor_sync(0xffffffffu, l_run[x], 2);
    }
    float* po = p.part_o + part * LAT_HEADS * p.V;
#pragma unroll
    for (int j = 0; j < LAT_MAX_NT; ++j)
        if (j < nt_w) {
            const int c = col0 + j * 8 + 2 * t4;
            *reinterpret_cast<float2*>(po + (size_t)(mt * 16 + g) * p.V + c) = make_float2(acc[j][0], acc[j][1]);
            *reinterpret_cast<float2*>(po + (size_t)(mt * 16 + g + 8) * p.V + c) = make_float2(acc[j][2], acc[j][3]);
        }
    if (ch == 0 && t4 == 0) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            p.part_ml[(part * LAT_HEADS + mt * 16 + g + 8 * x) * 2] = m_run[x];
            p.part_ml[(part * LAT_HEADS + mt * 16 + g + 8 * x) * 2 + 1] = l_run[x];
        }
    }
}

// out[tok, head, :] = sum_z o_z exp(m_z - m) / sum_z l_z exp(m_z - m), splits in order.  Grid (token, head);
// the splits' weights exp(m_z - m) / l are worked out once, into shared memory (splits floats).
__global__ void __launch_bounds__(128)
latent_combine_kernel(const float* part_o, const float* part_ml, bf16* out, int H, int V, int chunks, int splits) {
    extern __shared__ float wz[];                                  // [splits] maxima, then weights
    __shared__ float lz[128];                                       // the sums of 128 splits at a time
    __shared__ float m_all, inv_all;
    pdl_wait();
    pdl_launch_dependents();
    const int tok = blockIdx.x, head = blockIdx.y;
    const int hc = head / LAT_HEADS, r = head % LAT_HEADS;
    const size_t base = ((size_t)tok * chunks + hc) * splits;
    // all splits' maxima at once (one load a thread), then their common maximum and the weighted sum in split order
    for (int z = threadIdx.x; z < splits; z += blockDim.x) wz[z] = part_ml[((base + z) * LAT_HEADS + r) * 2];
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = -INFINITY;
        for (int z = 0; z < splits; ++z) m = fmaxf(m, wz[z]);
        m_all = m;
    }
    __syncthreads();
    const float m = m_all;
    float l = 0.f;
    for (int z0 = 0; z0 < splits; z0 += 128) {
        const int z = z0 + threadIdx.x;
        float e = 0.f, lv = 0.f;
        if (z < splits && wz[z] != -INFINITY) {
            e = expf(wz[z] - m);
            lv = part_ml[((base + z) * LAT_HEADS + r) * 2 + 1] * e;
        }
        __syncthreads();
        if (z < splits) wz[z] = e;
        lz[threadIdx.x] = lv;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int i = 0; i < min(128, splits - z0); ++i) l += lz[i];
        }
    }
    if (threadIdx.x == 0) inv_all = 1.0f / l;
    __syncthreads();
    const float inv = inv_all;
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        float o = 0.f;
        for (int z0 = 0; z0 < splits; z0 += 4) {                    // four splits' loads in flight, added in split order
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)                             // an empty split wrote no output: it is not read
                v[i] = (z0 + i < splits && wz[z0 + i] != 0.f) ? part_o[((base + z0 + i) * LAT_HEADS + r) * V + c] : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (z0 + i < splits) o += v[i] * wz[z0 + i];
        }
        out[((size_t)tok * H + head) * V + c] = __float2bfloat16_rn(o * inv);
    }
}

// Shared memory of the attention kernel for key rows of W elements.
static size_t latent_smem(int W) {
    return (size_t)(LAT_HEADS + 2 * LAT_TILE) * (W + LAT_PAD) * 2;
}

// q [n, H * W], cache [pages, 1, bs, W], out [n, H * V] (all bfloat16); part_o needs n * chunks * n_splits
// * 32 * V floats, part_ml the same with 2 in place of V (chunks = ceil(H / 32)); n_splits * split_keys
// must cover the longest context (with a window: the window and one tile); split_keys a multiple of 32.
RLLM_API int rllm_latent_decode_attention(const void* q, const void* cache, void* out, float* part_o, float* part_ml,
                                          const int* positions, const int* seq_ids, const int* block_table,
                                          int table_stride, int n, int H, int W, int V, int bs, float scale,
                                          float softcap, int split_keys, int n_splits, long long n_pages, int* err,
                                          int window, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || W % 16 || V % 64 || V <= 0 || V > 16 * LAT_MAX_NT || V > W || bs <= 0 || split_keys <= 0 ||
        split_keys % LAT_TILE || n_splits <= 0 || n_splits > 8192 || !part_o || !part_ml || softcap < 0.f || window < 0)
        return (int)cudaErrorInvalidValue;
    const size_t smem = latent_smem(W);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(latent_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    LatentParams p;
    p.q = (const bf16*)q; p.cache = (const bf16*)cache; p.part_o = part_o; p.part_ml = part_ml;
    p.positions = positions; p.seq_ids = seq_ids; p.block_table = block_table; p.table_stride = table_stride;
    p.n_pages = (int)(n_pages > 0x7fffffffLL ? 0x7fffffffLL : n_pages); p.err = err;
    p.H = H; p.W = W; p.V = V; p.bs = bs; p.split = split_keys; p.scale = scale; p.softcap = softcap; p.window = window;
    const int chunks = (H + LAT_HEADS - 1) / LAT_HEADS;
    int st = rllm_launch(latent_decode_kernel, dim3(n, chunks, n_splits), dim3(128), smem, stream, p);
    if (st) return st;
    return rllm_launch(latent_combine_kernel, dim3(n, H), dim3(128), (size_t)n_splits * sizeof(float), stream, (const float*)part_o,
                       (const float*)part_ml, (bf16*)out, H, V, chunks, n_splits);
}

RLLM_PACKED(rllm_latent_decode_attention)
