// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16),
// for head sizes 64 and 128.  Softmax runs in 32-bit with the scale applied
// after the dot product (crates/nncpu/src/kernels/scalar.rs:444-548), online
// over blocks of keys, and partial results are merged in key order like the
// reference's block partials (crates/nncpu/src/kernels/scalar.rs:521-548,
// crates/nncpu/src/model/forward.rs:174-190).
//
// Both kernels bring keys and values page by page (64 keys of one head) into
// shared memory with cp.async, several pages in flight, rows swizzled so that
// ldmatrix reads them without bank conflicts:
//   * prefill: one block per (64 consecutive new tokens of a sequence, head),
//     four warps of 16 query rows; causal and window masks per row;
//   * decode: one block per (token, key/value head, split of its pages).  With
//     one query per head the products are turned around so that the 16
//     tensor-core rows are keys and the columns are the query heads that share
//     the key/value head (grouped-query attention reads each key once for all
//     of them); the four warps each take 16 keys of a page.  Splits merge
//     inside a thread-block cluster through distributed shared memory, or, for
//     more than 8 splits, through scratch memory and a second kernel.

#include <math.h>
#include <mutex>

#define NN_LIB attention_mma
#include "common.cuh"

namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t smem_u32_(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t cluster_rank_() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier_() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32_(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Merges the splits of every (token, head) in split order.  grid = (n_heads, n_tok), HD threads.
template <int HD>
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             __nv_bfloat16* __restrict__ out, int n_heads, int n_kv, int n_splits) {
    const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    const int G = n_heads / n_kv, kvh = h / G, head = h % G;
    const size_t pb = ((size_t)t * n_kv + kvh) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[((pb + s) * G + head) * 2]);
    float o = 0.0f, l = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[((pb + s) * G + head) * 2];
        const float c = ms == -INFINITY ? 0.0f : exp2f(ms - m);
        o = fmaf(part_o[((pb + s) * G + head) * HD + d], c, o);
        l = fmaf(part_ml[((pb + s) * G + head) * 2 + 1], c, l);
    }
    out[((size_t)t * n_heads + h) * HD + d] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
}

// ---------------------------------------------------------------------------
// Prefill: any number of new tokens per sequence.  One block per (64
// consecutive new tokens of one sequence, head): four warps of 16 query rows
// each share the key and value tiles, which come page by page (64 keys) into
// shared memory with cp.async, two pages in flight, rows swizzled so that
// ldmatrix reads without bank conflicts.  grid = (tiles, n_heads).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Byte offset of the 16-byte chunk `chunk` of row `row` in a tile whose rows hold HD bfloat16:
// chunks are exchanged within groups of 8 by the row number, so 8 rows' equal chunks hit 8 bank groups.
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (HD * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(128, 3)
prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
               const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table, int bt_stride,
               const int* __restrict__ cu_seqlens, const int* __restrict__ tok_pos, __nv_bfloat16* __restrict__ out,
               int n_seqs, int n_heads, int n_kv, float scale2, int window) {
    constexpr int kTileBytes = kPage * HD * 2;           // one page of K or of V for one head
    constexpr int kChunks = HD / 8;                      // 16-byte chunks per row
    extern __shared__ __align__(128) uint8_t fa_smem[];  // [2 stages][K tile | V tile]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane & 3, r = lane >> 2;
    const int h = blockIdx.y;
    // tiles of 64 query rows, numbered within each sequence from its end (long spans first)
    int tile = blockIdx.x;
    int seq = -1, q0 = 0, q_end = 0;
    for (int b = 0; b < n_seqs; ++b) {
        const int a = cu_seqlens[b], e = cu_seqlens[b + 1];
        const int n_tiles = (e - a + 63) >> 6;
        if (tile < n_tiles) {
            seq = b;
            q0 = a + ((n_tiles - 1 - tile) << 6);
            q_end = e;
            break;
        }
        tile -= n_tiles;
    }
    if (seq < 0) return;
    const int n_rows = min(64, q_end - q0);
    const int pos0 = tok_pos[q0];                        // positions of a sequence's new tokens are consecutive
    const int key_hi = pos0 + n_rows - 1;                // the last row's last key
    const int key_lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int page_lo = key_lo / kPage, page_hi = key_hi / kPage;
    const int* table = block_table + (size_t)seq * bt_stride;
    const int kvh = h / (n_heads / n_kv);

    // this warp's rows: q0 + 16 * warp + r and + 8
    const int row_lo = 16 * warp + r, row_hi = row_lo + 8;
    const bool has_lo = row_lo < n_rows, has_hi = row_hi < n_rows;
    int lim_lo[2], lim_hi[2];
    lim_hi[0] = has_lo ? pos0 + row_lo : -1;
    lim_hi[1] = has_hi ? pos0 + row_hi : -1;
    lim_lo[0] = (window > 0 && lim_hi[0] + 1 > window) ? lim_hi[0] + 1 - window : 0;
    lim_lo[1] = (window > 0 && lim_hi[1] + 1 > window) ? lim_hi[1] + 1 - window : 0;
    const int warp_key_hi = pos0 + min(n_rows, 16 * warp + 16) - 1;   // nothing beyond this matters to the warp
    const int warp_key_lo = (window > 0 && pos0 + 16 * warp + 1 > window) ? pos0 + 16 * warp + 1 - window : 0;

    // query fragments in the layout the instruction asks for: 4-byte loads, once per block
    uint32_t qa[HD / 16][4];
    {
        const size_t stride = (size_t)n_heads * HD;
        const __nv_bfloat16* ql = q + (size_t)(q0 + row_lo) * stride + (size_t)h * HD;
        const __nv_bfloat16* qh = q + (size_t)(q0 + row_hi) * stride + (size_t)h * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qa[ks][0] = has_lo ? *reinterpret_cast<const uint32_t*>(ql + ks * 16 + 2 * c) : 0u;
            qa[ks][1] = has_hi ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * c) : 0u;
            qa[ks][2] = has_lo ? *reinterpret_cast<const uint32_t*>(ql + ks * 16 + 8 + 2 * c) : 0u;
            qa[ks][3] = has_hi ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 8 + 2 * c) : 0u;
        }
    }

    auto issue = [&](int page_idx, int stage) {
        const size_t base = ((size_t)table[page_idx] * n_kv + kvh) * (size_t)(kPage * HD);
        const uint32_t dst = smem_u32_(fa_smem) + stage * 2 * kTileBytes;
#pragma unroll
        for (int i = threadIdx.x; i < kPage * kChunks; i += 128) {
            const int row = i / kChunks, chunk = i % kChunks;
            cp_async16(dst + tile_off<HD>(row, chunk), k_pages + base + (size_t)row * HD + chunk * 8);
            cp_async16(dst + kTileBytes + tile_off<HD>(row, chunk), v_pages + base + (size_t)row * HD + chunk * 8);
        }
        cp_async_commit();
    };

    float o[HD / 8][4];
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    issue(page_lo, 0);
    for (int pg = page_lo; pg <= page_hi; ++pg) {
        const int stage = (pg - page_lo) & 1;
        if (pg + 1 <= page_hi) {
            issue(pg + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k_base = pg * kPage;
        if (k_base <= warp_key_hi && k_base + kPage - 1 >= warp_key_lo) {
            const uint32_t ks_addr = smem_u32_(fa_smem) + stage * 2 * kTileBytes;
            const uint32_t vs_addr = ks_addr + kTileBytes;
            // scores of 16 rows x 64 keys
            float s[8][4];
#pragma unroll
            for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int tp = 0; tp < 4; ++tp) {   // pairs of 8-key tiles
                    uint32_t b[4];
                    const int key = tp * 16 + (lane >> 4) * 8 + (lane & 7);
                    const int chunk = ks * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(b, ks_addr + tile_off<HD>(key, chunk));
                    mma_bf16(s[2 * tp], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
                    mma_bf16(s[2 * tp + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
                }
            }
            // scale, mask where the tile crosses a row's limits, running maximum
            const bool full = k_base >= max(lim_lo[0], lim_lo[1]) && has_hi && k_base + kPage - 1 <= lim_hi[0];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = e >> 1;
                    float v = s[t][e] * scale2;
                    if (!full) {
                        const int key = k_base + t * 8 + 2 * c + (e & 1);
                        if (key < lim_lo[row] || key > lim_hi[row]) v = -INFINITY;
                    }
                    s[t][e] = v;
                    mx[row] = fmaxf(mx[row], v);
                }
            float corr[2];
#pragma unroll
            for (int row = 0; row < 2; ++row) {
                mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
                mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
                const float m_new = fmaxf(m[row], mx[row]);
                corr[row] = m_new == -INFINITY ? 1.0f : fast_exp2(m[row] - m_new);
                m[row] = m_new;
            }
            float sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = e >> 1;
                    const float pv = m[row] == -INFINITY ? 0.0f : fast_exp2(s[t][e] - m[row]);
                    s[t][e] = pv;
                    sum[row] += pv;
                }
            l[0] = l[0] * corr[0] + sum[0];
            l[1] = l[1] * corr[1] + sum[1];
            if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
                for (int t = 0; t < HD / 8; ++t) {
                    o[t][0] *= corr[0]; o[t][1] *= corr[0]; o[t][2] *= corr[1]; o[t][3] *= corr[1];
                }
            }
            // weighted sum of the 64 value rows
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {       // 16 keys at a time
                const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {   // pairs of 8-lane tiles of the head
                    uint32_t b[4];
                    const int key = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int chunk = dp * 2 + (lane >> 4);
                    ldmatrix_x4_trans(b, vs_addr + tile_off<HD>(key, chunk));
                    mma_bf16(o[2 * dp], a0, a1, a2, a3, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the stage is free for the page after next
    }
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 1);
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 2);
        if (!(row == 0 ? has_lo : has_hi)) continue;
        const float inv = l[row] > 0.0f ? 1.0f / l[row] : 0.0f;
        __nv_bfloat16* dst = out + (size_t)(q0 + (row == 0 ? row_lo : row_hi)) * n_heads * HD + (size_t)h * HD;
#pragma unroll
        for (int t = 0; t < HD / 8; ++t)
            *reinterpret_cast<uint32_t*>(dst + t * 8 + 2 * c) = pack_bf16(o[t][2 * row] * inv, o[t][2 * row + 1] * inv);
    }
}

// ---------------------------------------------------------------------------
// Decode: one token per sequence.  How fast a block can stream its keys is set
// by how many bytes it has in flight, and registers hold only so many, so the
// pages go to shared memory: three pages per block in flight or in use.
//   S^T[16 keys, 8 heads]  = K[16 keys, HD]   . Q^T[HD, 8 heads]
//   O^T[HD,      8 heads] += V^T[HD, 16 keys] . P^T[16 keys, 8 heads]
// Keys fill the 16 tensor-core rows; the heads that share the key/value head are
// the 8 columns (a second column tile serves 9 to 16 heads).  P^T reaches the
// layout of a right-hand operand through movmatrix (an 8x8 transpose across the
// warp).  grid = (n_splits, n_kv, n_tok), 128 threads; splits are whole pages.
// ---------------------------------------------------------------------------
constexpr int kDecodeStages = 3;
constexpr int kMaxClusterSplits = 8;   // splits that merge inside a thread-block cluster (the portable cluster size)

// The decode kernel can start from the float32 q/k/v projections of its tokens instead of finished queries: every
// block then makes its own queries (per-head RMS norm, rotation: crates/nncpu/src/model/forward.rs:278-324), and the
// block whose keys end with the token itself also makes the token's key and value, appends them to the cache for the
// steps to come, and puts them into its copy of the page, where nobody else looks for them in this step.  The
// arithmetic is that of the separate kernel for norm, rotation and append, operation for operation.
struct FusedQK {
    const float* qkv;         // [n_tok, per_tok * HD]: the heads of q, then (if appended here) of k, then of v
    int per_tok;              // heads a token's row holds
    const void* q_gamma;      // per-head norm weights [HD], or null
    const void* k_gamma;
    int g_dt;
    float eps;
    const float2* cs;         // [n_tok, HD / 2] (cos, sin) of the tokens' positions, or null: no rotation
    __nv_bfloat16* k_pages;   // the cache, writable; null: the keys and values are another entry's, nothing is appended
    __nv_bfloat16* v_pages;
};

// One head's HD float32 values through norm (if gamma) and rotation (if cs) to bfloat16; a warp's job.  A lane holds
// HD / 32 neighbouring lanes of the head, so a rotation pair (i, i + HD / 2) sits in the lanes l and l ^ 16.
template <int HD>
__device__ __forceinline__ void finish_head(const float* __restrict__ src, const void* __restrict__ gamma, int g_dt, float eps,
                                            const float2* __restrict__ cs_row, __nv_bfloat16* __restrict__ dst, int lane) {
    constexpr int EPL = HD / 32;
    float x[EPL];
    if (EPL == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + lane * EPL);
        x[0] = v.x; x[1] = v.y; x[2 % EPL] = v.z; x[3 % EPL] = v.w;
    } else {
        const float2 v = *reinterpret_cast<const float2*>(src + lane * EPL);
        x[0] = v.x; x[1] = v.y;
    }
    if (gamma) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) ss = fmaf(x[e], x[e], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)HD) + eps);
#pragma unroll
        for (int e = 0; e < EPL; ++e) x[e] = (x[e] * scale) * ld_f(gamma, lane * EPL + e, g_dt);
    }
    if (cs_row != nullptr) {
        const int i0 = (lane & 15) * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            const float2 c = cs_row[i0 + e];
            x[e] = lane < 16 ? c.x * x[e] - c.y * other : c.y * other + c.x * x[e];
        }
    }
    if (EPL == 4) {
        __nv_bfloat162 o[2] = {__floats2bfloat162_rn(x[0], x[1]), __floats2bfloat162_rn(x[2 % EPL], x[3 % EPL])};
        *reinterpret_cast<uint2*>(dst + lane * 4) = *reinterpret_cast<uint2*>(o);
    } else {
        *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(x[0], x[1]);
    }
}

template <int HD, int NT, bool kCluster, bool kFused>
__global__ void __launch_bounds__(128, 2)
decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                   const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int n_heads, int n_kv, float scale2,
                   int window, const FusedQK f) {
    constexpr int kTileBytes = kPage * HD * 2;
    constexpr int kChunks = HD / 8;
    constexpr int W = HD + 2;
    extern __shared__ __align__(128) uint8_t dsm[];  // stages of [K page | V page]; afterwards the merge buffers
    const int split = blockIdx.x, n_splits = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane & 3, r = lane >> 2;
    const int G = n_heads / n_kv;
    const int seq = tok_seq[t];
    const size_t out_row = (size_t)t * n_heads * HD + (size_t)kvh * G * HD;
    if (seq < 0) {  // padding: zeros (every block of a cluster takes this way out together)
        if (n_splits == 1 || split == 0)
            for (int i = threadIdx.x; i < G * HD; i += 128) out[out_row + i] = __float2bfloat16_rn(0.0f);
        if (n_splits > 1 && !kCluster) {
            const size_t pb = ((size_t)t * n_kv + kvh) * n_splits + split;
            for (int i = threadIdx.x; i < G * HD; i += 128) part_o[pb * G * HD + i] = 0.0f;
            for (int i = threadIdx.x; i < G * 2; i += 128) part_ml[pb * G * 2 + i] = (i & 1) ? 0.0f : -INFINITY;
        }
        return;
    }
    const int pos = tok_pos[t];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int p_first = first / kPage, p_last = pos / kPage;
    const int per = (p_last - p_first + n_splits) / n_splits;      // pages per split, rounded up
    const int p0 = p_first + split * per, p1 = min(p_last, p0 + per - 1);
    const int* table = block_table + (size_t)seq * bt_stride;

    auto issue = [&](int page_idx, int stage) {
        const size_t base = ((size_t)table[page_idx] * n_kv + kvh) * (size_t)(kPage * HD);
        const uint32_t dst = smem_u32_(dsm) + stage * 2 * kTileBytes;
#pragma unroll
        for (int i = threadIdx.x; i < kPage * kChunks; i += 128) {
            const int row = i / kChunks, chunk = i % kChunks;
            cp_async16(dst + tile_off<HD>(row, chunk), k_pages + base + (size_t)row * HD + chunk * 8);
            cp_async16(dst + kTileBytes + tile_off<HD>(row, chunk), v_pages + base + (size_t)row * HD + chunk * 8);
        }
    };
    // two pages ahead; an empty commit keeps the group count in step when there is nothing to fetch
    if (p0 <= p1) issue(p0, 0);
    cp_async_commit();
    if (p0 + 1 <= p1) issue(p0 + 1, 1);
    cp_async_commit();

    // Started from the projections: this block's queries, and, in the block whose pages end with the token's own
    // position, the token's key and value (appended to the cache for later steps; for this step they are put into
    // the block's copy of the page when that has arrived).
    __shared__ __align__(16) __nv_bfloat16 q_s[kFused ? 16 * HD : 8];
    __shared__ __align__(16) __nv_bfloat16 kv_s[kFused ? 2 * HD : 8];
    const bool owner = kFused && f.k_pages != nullptr && p0 <= p_last && p_last <= p1;
    if constexpr (kFused) {
        const float* row = f.qkv + (size_t)t * f.per_tok * HD;
        const float2* cs_row = f.cs ? f.cs + (size_t)t * (HD / 2) : nullptr;
        for (int g = warp; g < G; g += 4)
            finish_head<HD>(row + (size_t)(kvh * G + g) * HD, f.q_gamma, f.g_dt, f.eps, cs_row, q_s + g * HD, lane);
        if (owner) {
            if (warp == 0)
                finish_head<HD>(row + (size_t)(n_heads + kvh) * HD, f.k_gamma, f.g_dt, f.eps, cs_row, kv_s, lane);
            if (warp == 1)
                finish_head<HD>(row + (size_t)(n_heads + n_kv + kvh) * HD, nullptr, 0, 0.0f, nullptr, kv_s + HD, lane);
        }
        __syncthreads();
        if (owner && threadIdx.x < 2 * kChunks) {
            const int which = threadIdx.x / kChunks, chunk = threadIdx.x % kChunks;
            __nv_bfloat16* page = (which ? f.v_pages : f.k_pages) +
                                  (((size_t)table[p_last] * n_kv + kvh) * kPage + pos % kPage) * (size_t)HD;
            *reinterpret_cast<uint4*>(page + chunk * 8) = *reinterpret_cast<const uint4*>(kv_s + which * HD + chunk * 8);
        }
    }
    // queries of the heads 8 * tt + r as right-hand operands: (lanes 2c, 2c + 1) and (2c + 8, 2c + 9) of each 16
    uint32_t qb[NT][HD / 16][2];
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
        const bool ok = 8 * tt + r < G;
        const __nv_bfloat16* qrow = kFused ? q_s + (size_t)(8 * tt + r) * HD : q + out_row + (size_t)(8 * tt + r) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qb[tt][ks][0] = ok ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * c) : 0u;
            qb[tt][ks][1] = ok ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * c) : 0u;
        }
    }
    float o[NT][HD / 16][4];
    float m[NT][2], l[NT][2];
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) o[tt][i][0] = o[tt][i][1] = o[tt][i][2] = o[tt][i][3] = 0.0f;
        m[tt][0] = m[tt][1] = -INFINITY;
        l[tt][0] = l[tt][1] = 0.0f;
    }

    for (int pg = p0; pg <= p1; ++pg) {
        const int stage = (pg - p0) % kDecodeStages;
        cp_async_wait<1>();        // this thread's copies of page pg have landed
        __syncthreads();           // everybody's have, and everybody is done with the stage refilled next
        if (pg + 2 <= p1) issue(pg + 2, (pg + 2 - p0) % kDecodeStages);
        cp_async_commit();
        if (kFused && owner && pg == p_last) {
            // the token's own key and value take their row of the page that has just arrived
            if (threadIdx.x < 2 * kChunks) {
                const int which = threadIdx.x / kChunks, chunk = threadIdx.x % kChunks;
                *reinterpret_cast<uint4*>(dsm + stage * 2 * kTileBytes + which * kTileBytes + tile_off<HD>(pos % kPage, chunk)) =
                    *reinterpret_cast<const uint4*>(kv_s + which * HD + chunk * 8);
            }
            __syncthreads();
        }
        const int k0 = pg * kPage + 16 * warp;             // this warp's 16 keys of the page
        if (k0 > pos || k0 + 15 < first) continue;
        const uint32_t ks_addr = smem_u32_(dsm) + stage * 2 * kTileBytes;
        const uint32_t vs_addr = ks_addr + kTileBytes;
        const bool inside = k0 >= first && k0 + 15 <= pos;
        const bool lo_ok = inside || (k0 + r >= first && k0 + r <= pos);
        const bool hi_ok = inside || (k0 + r + 8 >= first && k0 + r + 8 <= pos);
        // S^T = K . Q^T : 16 keys x 8 heads per column tile
        float s[NT][4];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) s[tt][0] = s[tt][1] = s[tt][2] = s[tt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t a[4];
            const int key = 16 * warp + ((lane >> 3) & 1) * 8 + (lane & 7);
            ldmatrix_x4(a, ks_addr + tile_off<HD>(key, ks * 2 + (lane >> 4)));
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) mma_bf16(s[tt], a[0], a[1], a[2], a[3], qb[tt][ks][0], qb[tt][ks][1]);
        }
        uint32_t pb[NT][2];
        float corr[NT][2];
        bool rescale = false;
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
            float* sv = s[tt];
            sv[0] = lo_ok ? sv[0] * scale2 : -INFINITY;
            sv[1] = lo_ok ? sv[1] * scale2 : -INFINITY;
            sv[2] = hi_ok ? sv[2] * scale2 : -INFINITY;
            sv[3] = hi_ok ? sv[3] * scale2 : -INFINITY;
            float mx0 = fmaxf(sv[0], sv[2]), mx1 = fmaxf(sv[1], sv[3]);
#pragma unroll
            for (int sh = 4; sh <= 16; sh <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
            }
            const float m0 = fmaxf(m[tt][0], mx0), m1 = fmaxf(m[tt][1], mx1);
            corr[tt][0] = m0 == -INFINITY ? 1.0f : fast_exp2(m[tt][0] - m0);
            corr[tt][1] = m1 == -INFINITY ? 1.0f : fast_exp2(m[tt][1] - m1);
            rescale = rescale || corr[tt][0] != 1.0f || corr[tt][1] != 1.0f;
            m[tt][0] = m0;
            m[tt][1] = m1;
            const float e0 = m0 == -INFINITY ? 0.0f : fast_exp2(sv[0] - m0), e2 = m0 == -INFINITY ? 0.0f : fast_exp2(sv[2] - m0);
            const float e1 = m1 == -INFINITY ? 0.0f : fast_exp2(sv[1] - m1), e3 = m1 == -INFINITY ? 0.0f : fast_exp2(sv[3] - m1);
            l[tt][0] = l[tt][0] * corr[tt][0] + (e0 + e2);
            l[tt][1] = l[tt][1] * corr[tt][1] + (e1 + e3);
            pb[tt][0] = movmatrix_trans(pack_bf16(e0, e1));
            pb[tt][1] = movmatrix_trans(pack_bf16(e2, e3));
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int tt = 0; tt < NT; ++tt)
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    o[tt][i][0] *= corr[tt][0]; o[tt][i][1] *= corr[tt][1];
                    o[tt][i][2] *= corr[tt][0]; o[tt][i][3] *= corr[tt][1];
                }
        }
        // O^T += V^T . P^T : 16 head lanes per row tile
#pragma unroll
        for (int dt = 0; dt < HD / 16; ++dt) {
            uint32_t a[4];
            const int key = 16 * warp + (lane >> 4) * 8 + (lane & 7);
            ldmatrix_x4_trans(a, vs_addr + tile_off<HD>(key, dt * 2 + ((lane >> 3) & 1)));
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) mma_bf16(o[tt][dt], a[0], a[1], a[2], a[3], pb[tt][0], pb[tt][1]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();   // the stages are free: they become the merge buffers
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int sh = 4; sh <= 16; sh <<= 1) l[tt][e] += __shfl_xor_sync(0xffffffffu, l[tt][e], sh);
    float* sm = reinterpret_cast<float*>(dsm);
    float* mine = sm + (size_t)warp * G * W;
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int head = 8 * tt + 2 * c + e;
            if (head < G) {
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    mine[head * W + i * 16 + r] = o[tt][i][e];
                    mine[head * W + i * 16 + r + 8] = o[tt][i][2 + e];
                }
                if (r == 0) {
                    mine[head * W + HD] = m[tt][e];
                    mine[head * W + HD + 1] = l[tt][e];
                }
            }
        }
    __syncthreads();
    const size_t pbase = ((size_t)t * n_kv + kvh) * n_splits + split;
    float* merged = sm + (size_t)4 * G * W;
    for (int i = threadIdx.x; i < G * HD; i += 128) {
        const int head = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm[(w * G + head) * W + HD]);
        float oo = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm[(w * G + head) * W + HD];
            const float cw = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
            oo = fmaf(sm[(w * G + head) * W + d], cw, oo);
            ll = fmaf(sm[(w * G + head) * W + HD + 1], cw, ll);
        }
        if (n_splits == 1) {
            out[out_row + i] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
        } else if (kCluster) {
            merged[head * W + d] = oo;
            if (d == 0) {
                merged[head * W + HD] = mm;
                merged[head * W + HD + 1] = ll;
            }
        } else {
            part_o[pbase * G * HD + i] = oo;
            if (d == 0) {
                part_ml[(pbase * G + head) * 2] = mm;
                part_ml[(pbase * G + head) * 2 + 1] = ll;
            }
        }
    }
    if (kCluster && n_splits > 1) {
        cluster_barrier_();   // every split's result is in its block's shared memory
        const int total = G * HD, share = (total + n_splits - 1) / n_splits;
        const int rank = (int)cluster_rank_();
        for (int i = rank * share + threadIdx.x; i < min(total, (rank + 1) * share); i += 128) {
            const int head = i / HD, d = i % HD;
            // all the loads from the other blocks' shared memory are issued before the first is used: one trip
            // through the cluster, not one per split
            float ms[kMaxClusterSplits], os[kMaxClusterSplits], ls[kMaxClusterSplits];
#pragma unroll
            for (int sp = 0; sp < kMaxClusterSplits; ++sp) {
                if (sp < n_splits) {
                    ms[sp] = ld_cluster_(merged + head * W + HD, sp);
                    os[sp] = ld_cluster_(merged + head * W + d, sp);
                    ls[sp] = ld_cluster_(merged + head * W + HD + 1, sp);
                }
            }
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < kMaxClusterSplits; ++sp)
                if (sp < n_splits) mm = fmaxf(mm, ms[sp]);
            float oo = 0.0f, ll = 0.0f;
#pragma unroll
            for (int sp = 0; sp < kMaxClusterSplits; ++sp) {
                if (sp < n_splits) {
                    const float cs = ms[sp] == -INFINITY ? 0.0f : exp2f(ms[sp] - mm);
                    oo = fmaf(os[sp], cs, oo);
                    ll = fmaf(ls[sp], cs, ll);
                }
            }
            out[out_row + i] = __float2bfloat16_rn(ll > 0.0f ? oo / ll : 0.0f);
        }
        cluster_barrier_();   // no block leaves while its result may still be read
    }
}

template <int HD>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int bt_stride,
                  const int* tok_seq, const int* tok_pos, void* out, float* scratch, int n_tok, int n_heads, int n_kv,
                  float scale, int window, int n_splits, cudaStream_t stream, const FusedQK* fused = nullptr) {
    using Kernel = void (*)(const __nv_bfloat16*, const __nv_bfloat16*, const __nv_bfloat16*, const int*, int, const int*,
                            const int*, __nv_bfloat16*, float*, float*, int, int, float, int, const FusedQK);
    const int G = n_heads / n_kv;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tok * n_kv * n_splits * G * HD : nullptr;
    // without scratch the splits merge inside a cluster (the caller checked n_splits <= 8)
    const bool cluster = scratch == nullptr && n_splits > 1;
    const Kernel plain = cluster ? (G <= 8 ? (Kernel)decode_kernel<HD, 1, true, false> : (Kernel)decode_kernel<HD, 2, true, false>)
                                 : (G <= 8 ? (Kernel)decode_kernel<HD, 1, false, false> : (Kernel)decode_kernel<HD, 2, false, false>);
    const Kernel from_qkv = cluster ? (G <= 8 ? (Kernel)decode_kernel<HD, 1, true, true> : (Kernel)decode_kernel<HD, 2, true, true>)
                                    : (G <= 8 ? (Kernel)decode_kernel<HD, 1, false, true> : (Kernel)decode_kernel<HD, 2, false, true>);
    const Kernel kernel = fused ? from_qkv : plain;
    const FusedQK f = fused ? *fused : FusedQK{};
    const size_t stages = (size_t)kDecodeStages * 2 * kPage * HD * 2;
    const size_t merge = (size_t)5 * G * (HD + 2) * sizeof(float);
    const size_t smem = stages > merge ? stages : merge;
    static bool configured[8][64] = {};
    if (first_use_on_this_device(configured[(fused ? 4 : 0) + (cluster ? 2 : 0) + (G <= 8 ? 0 : 1)])) {
        const cudaError_t e = cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)(stages > (size_t)5 * 16 * (HD + 2) * 4 ? stages : (size_t)5 * 16 * (HD + 2) * 4));
        NN_CHECK(e == cudaSuccess, "attention decode: cannot reserve shared memory: %s", cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_splits, n_kv, n_tok);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)n_splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cluster ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                                             (const __nv_bfloat16*)v_pages, block_table, bt_stride, tok_seq, tok_pos,
                                             (__nv_bfloat16*)out, part_o, part_ml, n_heads, n_kv, scale * kLog2e, window, f);
    NN_CHECK(e == cudaSuccess, "attention decode (%d splits%s): launch failed: %s", n_splits, cluster ? ", cluster" : "",
             cudaGetErrorString(e));
    if (n_splits > 1 && !cluster) {
        merge_kernel<HD><<<dim3(n_heads, n_tok), HD, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, n_heads, n_kv,
                                                                  n_splits);
        NN_LAUNCH_OK("attention merge");
    }
    return 0;
}

template <int HD>
int launch_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int bt_stride,
                   const int* cu_seqlens, const int* tok_pos, void* out, int n_tok, int n_seqs, int n_heads, int n_kv,
                   float scale, int window, cudaStream_t stream) {
    const int max_tiles = n_tok / 64 + n_seqs;
    constexpr int smem = 2 * 2 * kPage * HD * 2;
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        NN_CHECK(e == cudaSuccess, "attention prefill: cannot reserve shared memory: %s", cudaGetErrorString(e));
    }
    dim3 grid(max_tiles, n_heads);
    prefill_kernel<HD><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                                                 (const __nv_bfloat16*)v_pages, block_table, bt_stride, cu_seqlens,
                                                 tok_pos, (__nv_bfloat16*)out, n_seqs, n_heads, n_kv, scale * kLog2e,
                                                 window);
    NN_LAUNCH_OK("attention prefill");
    return 0;
}

}  // namespace

// Whether the tensor-core attention kernels take these sizes (bfloat16 q, cache and output assumed).
extern "C" int nncpu_attention_mma_supported(int n_heads, int n_kv, int hd) {
    return (hd == 64 || hd == 128) && n_kv > 0 && n_heads % n_kv == 0 && n_heads / n_kv <= 16;
}

// Floats of scratch the decode kernel needs for n_tok tokens cut into n_splits splits (0 for one split).
extern "C" long nncpu_attention_decode_scratch_floats(int n_tok, int n_heads, int n_kv, int hd, int n_splits) {
    if (n_splits <= 1) return 0;
    const long G = n_heads / n_kv;
    return (long)n_tok * n_kv * n_splits * G * (hd + 2);
}

// One token per sequence: token t belongs to sequence tok_seq[t] (negative: padding) and sits at
// position tok_pos[t]; its keys 0..tok_pos[t] (or the last `window` of them) are in the cache.
extern "C" int nncpu_attention_decode_mma(const void* q, const void* k_pages, const void* v_pages,
                                          const int* block_table, int bt_stride, const int* tok_seq,
                                          const int* tok_pos, void* out, float* scratch, long scratch_floats,
                                          int n_tok, int n_heads, int n_kv, int hd, float scale, int window,
                                          int n_splits, void* stream) {
    NN_CHECK(nncpu_attention_mma_supported(n_heads, n_kv, hd),
             "attention (tensor cores): %d heads over %d key/value heads of size %d is not supported "
             "(head size 64 or 128, at most 16 heads per key/value head)", n_heads, n_kv, hd);
    NN_CHECK(n_tok >= 0 && n_splits >= 1 && n_splits <= 65535 && window >= 0, "attention decode: %d tokens, %d splits",
             n_tok, n_splits);
    if (scratch == nullptr && n_splits > 1)
        NN_CHECK(n_splits <= 8, "attention decode: %d splits without scratch (a cluster merges at most 8)", n_splits);
    else
        NN_CHECK(scratch_floats >= nncpu_attention_decode_scratch_floats(n_tok, n_heads, n_kv, hd, n_splits),
                 "attention decode: %ld floats of scratch, %ld needed", scratch_floats,
                 nncpu_attention_decode_scratch_floats(n_tok, n_heads, n_kv, hd, n_splits));
    if (n_tok == 0) return 0;
    if (hd == 64)
        return launch_decode<64>(q, k_pages, v_pages, block_table, bt_stride, tok_seq, tok_pos, out, scratch, n_tok,
                                 n_heads, n_kv, scale, window, n_splits, (cudaStream_t)stream);
    return launch_decode<128>(q, k_pages, v_pages, block_table, bt_stride, tok_seq, tok_pos, out, scratch, n_tok,
                              n_heads, n_kv, scale, window, n_splits, (cudaStream_t)stream);
}

// The same from the float32 projections: qkv [n_tok, per_tok * hd] holds, per token, the heads of q and, if `append`,
// of k and v after them (per_tok = n_heads + 2 n_kv, else n_heads).  Every block makes its queries itself (per-head RMS
// norm with q_gamma if given, rotation by cos_sin [n_tok, hd / 2, 2] if given); with `append` the token's key (k_gamma,
// rotation) and value are made too, written to their row of the cache pages and used in this step.  Replaces the
// separate kernel for norm, rotation and append in a decode step; the arithmetic is the same.
extern "C" int nncpu_attention_decode_mma_from_qkv(const float* qkv, const void* q_gamma, const void* k_gamma, int g_dt,
                                                   float eps, const float* cos_sin, void* k_pages, void* v_pages,
                                                   int append, const int* block_table, int bt_stride,
                                                   const int* tok_seq, const int* tok_pos, void* out, float* scratch,
                                                   long scratch_floats, int n_tok, int n_heads, int n_kv, int hd,
                                                   float scale, int window, int n_splits, void* stream) {
    NN_CHECK(nncpu_attention_mma_supported(n_heads, n_kv, hd),
             "attention (tensor cores): %d heads over %d key/value heads of size %d is not supported "
             "(head size 64 or 128, at most 16 heads per key/value head)", n_heads, n_kv, hd);
    NN_CHECK(n_tok >= 0 && n_splits >= 1 && n_splits <= 65535 && window >= 0, "attention decode: %d tokens, %d splits",
             n_tok, n_splits);
    NN_CHECK(qkv != nullptr && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)cos_sin % 8) == 0 && ((uintptr_t)k_pages % 16) == 0 &&
                 ((uintptr_t)v_pages % 16) == 0,
             "attention decode (from projections): the projections and the cache must be 16-byte aligned, the rotation "
             "table 8-byte aligned");
    if (scratch == nullptr && n_splits > 1)
        NN_CHECK(n_splits <= 8, "attention decode: %d splits without scratch (a cluster merges at most 8)", n_splits);
    else
        NN_CHECK(scratch_floats >= nncpu_attention_decode_scratch_floats(n_tok, n_heads, n_kv, hd, n_splits),
                 "attention decode: %ld floats of scratch, %ld needed", scratch_floats,
                 nncpu_attention_decode_scratch_floats(n_tok, n_heads, n_kv, hd, n_splits));
    if (n_tok == 0) return 0;
    FusedQK f{};
    f.qkv = qkv;
    f.per_tok = append ? n_heads + 2 * n_kv : n_heads;
    f.q_gamma = q_gamma; f.k_gamma = k_gamma; f.g_dt = g_dt; f.eps = eps;
    f.cs = (const float2*)cos_sin;
    f.k_pages = append ? (__nv_bfloat16*)k_pages : nullptr;
    f.v_pages = append ? (__nv_bfloat16*)v_pages : nullptr;
    if (hd == 64)
        return launch_decode<64>(nullptr, k_pages, v_pages, block_table, bt_stride, tok_seq, tok_pos, out, scratch, n_tok,
                                 n_heads, n_kv, scale, window, n_splits, (cudaStream_t)stream, &f);
    return launch_decode<128>(nullptr, k_pages, v_pages, block_table, bt_stride, tok_seq, tok_pos, out, scratch, n_tok,
                              n_heads, n_kv, scale, window, n_splits, (cudaStream_t)stream, &f);
}

// Any mix of new tokens per sequence: sequence b brings the flat tokens cu_seqlens[b] .. cu_seqlens[b + 1] - 1
// at consecutive positions starting at tok_pos[cu_seqlens[b]]; their keys are already in the cache.
extern "C" int nncpu_attention_prefill_mma(const void* q, const void* k_pages, const void* v_pages,
                                           const int* block_table, int bt_stride, const int* cu_seqlens,
                                           const int* tok_pos, void* out, int n_tok, int n_seqs, int n_heads,
                                           int n_kv, int hd, float scale, int window, void* stream) {
    NN_CHECK(nncpu_attention_mma_supported(n_heads, n_kv, hd),
             "attention (tensor cores): %d heads over %d key/value heads of size %d is not supported "
             "(head size 64 or 128, at most 16 heads per key/value head)", n_heads, n_kv, hd);
    NN_CHECK(n_tok >= 0 && n_seqs >= 0 && window >= 0, "attention prefill: %d tokens of %d sequences", n_tok, n_seqs);
    if (n_tok == 0 || n_seqs == 0) return 0;
    if (hd == 64)
        return launch_prefill<64>(q, k_pages, v_pages, block_table, bt_stride, cu_seqlens, tok_pos, out, n_tok, n_seqs,
                                  n_heads, n_kv, scale, window, (cudaStream_t)stream);
    return launch_prefill<128>(q, k_pages, v_pages, block_table, bt_stride, cu_seqlens, tok_pos, out, n_tok, n_seqs,
                               n_heads, n_kv, scale, window, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Decode attention for callers that cannot bring scratch memory.
// Declared in attention_mma_static.h; it has no counterpart in the reference.
//
// nncpu_attention_decode_mma merges its key splits through a scratch buffer
// that the caller allocates.  Some callers have no way to allocate device
// memory: a host that has already given every free byte of the GPU to its own
// cache and weight pools, so that cudaMalloc fails; a plugin or foreign-language
// binding that is handed raw device pointers and owns no allocator; a real-time
// loop that must not enter the driver's allocator because that can stall the
// whole device.  For them the scratch lives in this library's own image: a
// file-scope __device__ array of kStaticScratchFloats floats (4 MiB), which
// every GPU that loads the library holds until the process exits.
//
// In host code the array's name is only a host-side stand-in for the device
// symbol, not a device address, so the address is looked up with
// cudaGetSymbolAddress: once per device, with that device current, on the
// first call made on that device.  That first call does this set-up; make it
// before any stream capture begins.  The entry point calls no cudaMalloc,
// cudaFree or other allocating routine.
//
// All calls on a device share the one array, and the array keeps what the last
// call left in it.  Nothing in it has to start at zero: every split writes its
// whole partial result (a split without keys writes "no keys") before the
// merge kernel of the same call reads it, so stale contents are never read.
// Two calls that overlap on the GPU (different streams, or graphs replayed
// side by side) would write the same floats and race: keep calls on a device
// in one stream, or order them yourself.
// ---------------------------------------------------------------------------
namespace {

constexpr long kStaticScratchFloats = 1l << 20;  // 4 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_lock;
float* g_static_ptr[kMaxDevices] = {};

// The device address of g_static_scratch on the current device.
int static_scratch(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    NN_CHECK(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, "attention decode (static scratch): no usable current device (%s)",
             cudaGetErrorString(e));
    std::lock_guard<std::mutex> g(g_static_lock);
    if (g_static_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        NN_CHECK(e == cudaSuccess && p != nullptr, "attention decode (static scratch): cudaGetSymbolAddress failed on device %d: %s", dev,
                 cudaGetErrorString(e));
        g_static_ptr[dev] = static_cast<float*>(p);
    }
    *ptr = g_static_ptr[dev];
    return 0;
}

}  // namespace

extern "C" long nncpu_attention_decode_mma_static_max_floats() { return kStaticScratchFloats; }

extern "C" int nncpu_attention_decode_mma_static(const void* q, const void* k_pages, const void* v_pages,
                                                 const int* block_table, int bt_stride, const int* tok_seq,
                                                 const int* tok_pos, void* out, int n_tok, int n_heads, int n_kv,
                                                 int hd, float scale, int window, int n_splits, void* stream) {
    NN_CHECK(nncpu_attention_mma_supported(n_heads, n_kv, hd),
             "attention (tensor cores): %d heads over %d key/value heads of size %d is not supported "
             "(head size 64 or 128, at most 16 heads per key/value head)", n_heads, n_kv, hd);
    NN_CHECK(n_tok >= 0 && n_splits >= 1 && n_splits <= 65535, "attention decode (static scratch): %d tokens, %d splits", n_tok,
             n_splits);
    const long need = nncpu_attention_decode_scratch_floats(n_tok, n_heads, n_kv, hd, n_splits);
    NN_CHECK(need <= kStaticScratchFloats,
             "attention decode (static scratch): %d tokens x %d key/value heads x %d splits need %ld floats of scratch, "
             "the built-in buffer holds %ld; use fewer splits or tokens per call, or nncpu_attention_decode_mma with "
             "scratch of your own", n_tok, n_kv, n_splits, need, kStaticScratchFloats);
    float* scratch = nullptr;
    if (int e = static_scratch(&scratch)) return e;
    return nncpu_attention_decode_mma(q, k_pages, v_pages, block_table, bt_stride, tok_seq, tok_pos, out, scratch,
                                      kStaticScratchFloats, n_tok, n_heads, n_kv, hd, scale, window, n_splits, stream);
}
