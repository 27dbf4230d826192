// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16),
// for head sizes 64 and 128.  Softmax runs in 32-bit with the scale applied
// after the dot product (crates/nncpu/src/kernels/scalar.rs:444-548), online
// over groups of 16 keys, and partial results are merged in key order like the
// reference's block partials (crates/nncpu/src/kernels/scalar.rs:521-548,
// crates/nncpu/src/model/forward.rs:174-190).
//
// Keys and values go from global memory (or L2) straight into the registers
// of the warp that multiplies them: no shared-memory staging.  That works
// because a matrix product does not care in which order its inner index runs
// as long as both operands agree:
//   * scores: a lane loads 16 bytes (8 lanes of the head) of its key row and
//     of its query row at the same offsets, and feeds them to the tensor core
//     as if they were the 4 lanes the fragment layout asks for;
//   * weighted sum: a lane loads 16 bytes of 4 value rows and interleaves them
//     with byte permutes into the "two consecutive keys per register" form.
//
// Two kernels share the inner loop:
//   * decode: one block per (token, key/value head, split of its keys); the 16
//     tensor-core rows hold the query heads that share the key/value head
//     (grouped-query attention reads each key once for all of them); the
//     block's four warps take alternate 16-key groups; splits are merged by a
//     second kernel through a scratch buffer.
//   * prefill: one warp per (16 consecutive tokens of a sequence, head).

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

__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ uint32_t smem_u32_(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// What one warp carries through its keys: 16 rows x HD output lanes, the running maximum (in the
// log2 domain, scale folded in) and the running sum of each of its two rows per lane.
template <int HD>
struct Acc {
    float o[HD / 8][4];
    float m[2], l[2];
    __device__ void init() {
#pragma unroll
        for (int t = 0; t < HD / 8; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[t][e] = 0.0f;
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.0f;
    }
};

// Query fragments of the rows (lane / 4) and (lane / 4 + 8); a null row gives zeros.
template <int HD>
__device__ __forceinline__ void load_q(uint32_t (&qa)[HD / 16][4], const __nv_bfloat16* row_lo,
                                       const __nv_bfloat16* row_hi, int lane) {
    const int c = lane & 3;
#pragma unroll
    for (int j = 0; j < HD / 32; ++j) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        const uint4 lo = row_lo ? ld16(row_lo + (c + 4 * j) * 8) : z;
        const uint4 hi = row_hi ? ld16(row_hi + (c + 4 * j) * 8) : z;
        qa[2 * j][0] = lo.x; qa[2 * j][2] = lo.y; qa[2 * j][1] = hi.x; qa[2 * j][3] = hi.y;
        qa[2 * j + 1][0] = lo.z; qa[2 * j + 1][2] = lo.w; qa[2 * j + 1][1] = hi.z; qa[2 * j + 1][3] = hi.w;
    }
}

struct Pages {
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    const int* table;  // page ids of this sequence
    int n_kv, kvh;
    template <int HD>
    __device__ __forceinline__ size_t row(int key) const {
        return (((size_t)table[key / kPage] * n_kv + kvh) * kPage + key % kPage) * HD;
    }
};

// Registers holding one group of 16 keys: two 8-key tiles of K, four value rows per lane.
template <int HD>
struct Group {
    uint4 k[2][HD / 32];
    uint4 v[4][HD / 64];
};

// Loads the group that starts at key k0 (a multiple of 16).  Keys outside [key_lo, key_hi] are
// not touched (their pages may be gone) and read as zeros.
template <int HD>
__device__ __forceinline__ void load_group(Group<HD>& g, const Pages& pg, int k0, int key_lo, int key_hi, int lane) {
    const int c = lane & 3, r = lane >> 2;
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int key = k0 + 8 * t + r;
        const bool ok = key >= key_lo && key <= key_hi;
        const __nv_bfloat16* p = pg.k + (ok ? pg.row<HD>(key) : 0);
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) g.k[t][j] = ok ? ld16(p + (c + 4 * j) * 8) : z;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int key = k0 + 2 * c + (i & 1) + 8 * (i >> 1);
        const bool ok = key >= key_lo && key <= key_hi;
        const __nv_bfloat16* p = pg.v + (ok ? pg.row<HD>(key) : 0);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) g.v[i][h] = ok ? ld16(p + h * 64 + r * 8) : z;
    }
}

// One group of 16 keys starting at k0 into the accumulators.  Row `e` (0: lane / 4, 1: lane / 4 + 8)
// sees the keys lo[e] .. hi[e]; scale2 = scale * log2(e).
template <int HD>
__device__ __forceinline__ void consume_group(Acc<HD>& acc, const uint32_t (&qa)[HD / 16][4], const Group<HD>& g,
                                              int k0, const int (&lo)[2], const int (&hi)[2], float scale2,
                                              int lane) {
    const int c = lane & 3;
    float s[2][4];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.0f;
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) {
            mma_bf16(s[t], qa[2 * j][0], qa[2 * j][1], qa[2 * j][2], qa[2 * j][3], g.k[t][j].x, g.k[t][j].y);
            mma_bf16(s[t], qa[2 * j + 1][0], qa[2 * j + 1][1], qa[2 * j + 1][2], qa[2 * j + 1][3], g.k[t][j].z,
                     g.k[t][j].w);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = k0 + 8 * t + 2 * c + (e & 1), row = e >> 1;
            const bool ok = key >= lo[row] && key <= hi[row];
            s[t][e] = ok ? s[t][e] * scale2 : -INFINITY;
            mx[row] = fmaxf(mx[row], s[t][e]);
        }
    float corr[2];
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
        const float m_new = fmaxf(acc.m[row], mx[row]);
        corr[row] = m_new == -INFINITY ? 1.0f : exp2f(acc.m[row] - m_new);
        acc.m[row] = m_new;
    }
    uint32_t pa[4];
    {
        float p[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = e >> 1;
                p[t][e] = acc.m[row] == -INFINITY ? 0.0f : exp2f(s[t][e] - acc.m[row]);
            }
#pragma unroll
        for (int row = 0; row < 2; ++row)
            acc.l[row] = acc.l[row] * corr[row] + (p[0][2 * row] + p[0][2 * row + 1]) + (p[1][2 * row] + p[1][2 * row + 1]);
        pa[0] = pack_bf16(p[0][0], p[0][1]);
        pa[1] = pack_bf16(p[0][2], p[0][3]);
        pa[2] = pack_bf16(p[1][0], p[1][1]);
        pa[3] = pack_bf16(p[1][2], p[1][3]);
    }
#pragma unroll
    for (int h = 0; h < HD / 64; ++h)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float (&o)[4] = acc.o[h * 8 + e];
            o[0] *= corr[0]; o[1] *= corr[0]; o[2] *= corr[1]; o[3] *= corr[1];
            const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = __byte_perm(u4_get(g.v[0][h], e >> 1), u4_get(g.v[1][h], e >> 1), sel);
            const uint32_t b1 = __byte_perm(u4_get(g.v[2][h], e >> 1), u4_get(g.v[3][h], e >> 1), sel);
            mma_bf16(o, pa[0], pa[1], pa[2], pa[3], b0, b1);
        }
}

// Asks for the K and V rows of the group at k0 to be brought into L2: one 128-byte line per lane.
// Loads in registers bound how many bytes a warp can have in flight; prefetches do not.
template <int HD>
__device__ __forceinline__ void prefetch_group(const Pages& pg, int k0, int key_lo, int key_hi, int lane) {
    constexpr int kLinesPerRow = HD * 2 / 128;         // 2 for head size 128, 1 for 64
    const int key = k0 + lane / kLinesPerRow;
    if (lane < 16 * kLinesPerRow && key >= key_lo && key <= key_hi) {
        const size_t off = pg.row<HD>(key) + (size_t)(lane % kLinesPerRow) * 64;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pg.k + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pg.v + off));
    }
}

constexpr int kPrefetchAhead = 4;   // groups of 16 keys ahead of the one being loaded

// Runs the groups first_group, first_group + stride, ... that overlap [key_lo, key_hi].
template <int HD>
__device__ __forceinline__ void run_keys(Acc<HD>& acc, const uint32_t (&qa)[HD / 16][4], const Pages& pg, int key_lo,
                                         int key_hi, const int (&lo)[2], const int (&hi)[2], int first_group,
                                         int stride, float scale2, int lane) {
    const int last_group = key_hi >> 4;
    int gi = first_group;
    if (gi > last_group) return;
    Group<HD> cur, nxt;
#pragma unroll
    for (int a = 1; a <= kPrefetchAhead; ++a)
        if (gi + a * stride <= last_group) prefetch_group<HD>(pg, (gi + a * stride) << 4, key_lo, key_hi, lane);
    load_group<HD>(cur, pg, gi << 4, key_lo, key_hi, lane);
    while (true) {
        const int gn = gi + stride;
        const bool more = gn <= last_group;
        if (gn + kPrefetchAhead * stride <= last_group)
            prefetch_group<HD>(pg, (gn + kPrefetchAhead * stride) << 4, key_lo, key_hi, lane);
        if (more) load_group<HD>(nxt, pg, gn << 4, key_lo, key_hi, lane);
        consume_group<HD>(acc, qa, cur, gi << 4, lo, hi, scale2, lane);
        if (!more) break;
        cur = nxt;
        gi = gn;
    }
}

// The actual head lane of accumulator register (tile t, element e) for this lane.
template <int HD>
__device__ __forceinline__ int out_dim(int t, int e, int lane) {
    return (t >> 3) * 64 + (2 * (lane & 3) + (e & 1)) * 8 + (t & 7);
}

// ---------------------------------------------------------------------------
// Decode: one token per sequence.  grid = (n_splits, n_kv, n_tok), 128 threads.
//
// With one query per head there are only G = heads / kv-heads rows to fill a
// 16-row tensor-core tile, so the decode kernel turns the products around:
//   S^T[16 keys, 8 heads]  = K[16 keys, HD]      . Q^T[HD, 8 heads]
//   O^T[HD,      8 heads] += V^T[HD, 16 keys]    . P^T[16 keys, 8 heads]
// Keys fill the 16 rows, the heads that share the key/value head are the 8
// columns (a second column tile serves 9 to 16 heads).  P^T reaches the layout
// of a right-hand operand through movmatrix (an 8x8 transpose across the warp).
// ---------------------------------------------------------------------------
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

// Registers of one group of 16 keys for the decode formulation: key rows (lane / 4) and (lane / 4 + 8)
// of K, and the value rows of the keys 2c, 2c + 1, 2c + 8, 2c + 9 (c = lane % 4).
template <int HD>
struct DGroup {
    uint4 k_lo[HD / 32], k_hi[HD / 32];
    uint4 v[4][HD / 64];
};

template <int HD>
__device__ __forceinline__ void d_load_group(DGroup<HD>& g, const Pages& pg, int k0, int key_lo, int key_hi, int lane) {
    const int c = lane & 3, r = lane >> 2;
    const uint4 z = make_uint4(0, 0, 0, 0);
    // the 16 keys of a group lie in one page
    const size_t base = (((size_t)pg.table[k0 / kPage] * pg.n_kv + pg.kvh) * kPage + k0 % kPage) * HD;
    const __nv_bfloat16* kb = pg.k + base;
    const __nv_bfloat16* vb = pg.v + base;
    const bool inside = k0 >= key_lo && k0 + 15 <= key_hi;
    if (inside) {
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) {
            g.k_lo[j] = ld16(kb + (size_t)r * HD + (c + 4 * j) * 8);
            g.k_hi[j] = ld16(kb + (size_t)(r + 8) * HD + (c + 4 * j) * 8);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int h = 0; h < HD / 64; ++h)
                g.v[i][h] = ld16(vb + (size_t)(2 * c + (i & 1) + 8 * (i >> 1)) * HD + h * 64 + r * 8);
    } else {
        const bool lo_ok = k0 + r >= key_lo && k0 + r <= key_hi, hi_ok = k0 + r + 8 >= key_lo && k0 + r + 8 <= key_hi;
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) {
            g.k_lo[j] = lo_ok ? ld16(kb + (size_t)r * HD + (c + 4 * j) * 8) : z;
            g.k_hi[j] = hi_ok ? ld16(kb + (size_t)(r + 8) * HD + (c + 4 * j) * 8) : z;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rel = 2 * c + (i & 1) + 8 * (i >> 1);
            const bool ok = k0 + rel >= key_lo && k0 + rel <= key_hi;
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) g.v[i][h] = ok ? ld16(vb + (size_t)rel * HD + h * 64 + r * 8) : z;
        }
    }
}

// Per-lane state of the decode formulation for NT column tiles of 8 heads: the lane's two heads
// of each tile are 8 * t + 2c and 8 * t + 2c + 1.
template <int HD, int NT>
struct DAcc {
    float o[NT][HD / 16][4];  // row tile (h, e): [0..1] head lane (h * 64 + r * 8 + e), [2..3] head lane (.. + 4)
    float m[NT][2], l[NT][2];
};

template <int HD, int NT>
__device__ __forceinline__ void d_consume_group(DAcc<HD, NT>& acc, const uint4 (&q)[NT][HD / 32], const DGroup<HD>& g,
                                                int k0, int key_lo, int key_hi, float scale2, int lane) {
    const int c = lane & 3, r = lane >> 2;
    const bool inside = k0 >= key_lo && k0 + 15 <= key_hi;
    const bool lo_ok = inside || (k0 + r >= key_lo && k0 + r <= key_hi);
    const bool hi_ok = inside || (k0 + r + 8 >= key_lo && k0 + r + 8 <= key_hi);
    uint32_t pb[NT][2];
    bool rescale = false;
    float corr[NT][2];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) {
            mma_bf16(s, g.k_lo[j].x, g.k_hi[j].x, g.k_lo[j].y, g.k_hi[j].y, q[t][j].x, q[t][j].y);
            mma_bf16(s, g.k_lo[j].z, g.k_hi[j].z, g.k_lo[j].w, g.k_hi[j].w, q[t][j].z, q[t][j].w);
        }
        // s[0], s[1]: key k0 + r, heads 2c, 2c + 1;  s[2], s[3]: key k0 + r + 8
        s[0] = lo_ok ? s[0] * scale2 : -INFINITY;
        s[1] = lo_ok ? s[1] * scale2 : -INFINITY;
        s[2] = hi_ok ? s[2] * scale2 : -INFINITY;
        s[3] = hi_ok ? s[3] * scale2 : -INFINITY;
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
        }
        const float m0 = fmaxf(acc.m[t][0], mx0), m1 = fmaxf(acc.m[t][1], mx1);
        corr[t][0] = m0 == -INFINITY ? 1.0f : fast_exp2(acc.m[t][0] - m0);
        corr[t][1] = m1 == -INFINITY ? 1.0f : fast_exp2(acc.m[t][1] - m1);
        rescale = rescale || corr[t][0] != 1.0f || corr[t][1] != 1.0f;
        acc.m[t][0] = m0;
        acc.m[t][1] = m1;
        const float p0 = m0 == -INFINITY ? 0.0f : fast_exp2(s[0] - m0), p2 = m0 == -INFINITY ? 0.0f : fast_exp2(s[2] - m0);
        const float p1 = m1 == -INFINITY ? 0.0f : fast_exp2(s[1] - m1), p3 = m1 == -INFINITY ? 0.0f : fast_exp2(s[3] - m1);
        acc.l[t][0] = acc.l[t][0] * corr[t][0] + (p0 + p2);
        acc.l[t][1] = acc.l[t][1] * corr[t][1] + (p1 + p3);
        // (key, head pair) -> (head, key pair): the right-hand operand of the second product
        pb[t][0] = movmatrix_trans(pack_bf16(p0, p1));
        pb[t][1] = movmatrix_trans(pack_bf16(p2, p3));
    }
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) {
                acc.o[t][i][0] *= corr[t][0]; acc.o[t][i][1] *= corr[t][1];
                acc.o[t][i][2] *= corr[t][0]; acc.o[t][i][3] *= corr[t][1];
            }
    }
#pragma unroll
    for (int h = 0; h < HD / 64; ++h)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
            const uint32_t a0 = __byte_perm(u4_get(g.v[0][h], e >> 1), u4_get(g.v[1][h], e >> 1), sel);
            const uint32_t a1 = __byte_perm(u4_get(g.v[0][h], 2 + (e >> 1)), u4_get(g.v[1][h], 2 + (e >> 1)), sel);
            const uint32_t a2 = __byte_perm(u4_get(g.v[2][h], e >> 1), u4_get(g.v[3][h], e >> 1), sel);
            const uint32_t a3 = __byte_perm(u4_get(g.v[2][h], 2 + (e >> 1)), u4_get(g.v[3][h], 2 + (e >> 1)), sel);
#pragma unroll
            for (int t = 0; t < NT; ++t) mma_bf16(acc.o[t][h * 4 + e], a0, a1, a2, a3, pb[t][0], pb[t][1]);
        }
}

template <int HD, int NT>
__global__ void __launch_bounds__(128, 2)
decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
              const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table, int bt_stride,
              const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, __nv_bfloat16* __restrict__ out,
              float* __restrict__ part_o, float* __restrict__ part_ml, int n_heads, int n_kv, float scale2,
              int window) {
    extern __shared__ float sm[];  // [4 warps][G rows][HD + 2]
    const int split = blockIdx.x, n_splits = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = n_heads / n_kv;  // at most 8 * NT
    const int seq = tok_seq[t];
    const size_t out_row = (size_t)t * n_heads * HD + (size_t)kvh * G * HD;
    if (seq < 0) {  // padding: zeros
        if (n_splits == 1 || split == 0)
            for (int i = threadIdx.x; i < G * HD; i += 128) out[out_row + i] = __float2bfloat16_rn(0.0f);
        if (n_splits > 1) {
            const size_t pb = ((size_t)t * n_kv + kvh) * n_splits + split;
            for (int i = threadIdx.x; i < G * HD; i += 128) part_o[pb * G * HD + i] = 0.0f;
            for (int i = threadIdx.x; i < G * 2; i += 128) part_ml[pb * G * 2 + i] = (i & 1) ? 0.0f : -INFINITY;
        }
        return;
    }
    const int pos = tok_pos[t];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    // this split's keys: whole 16-key groups, the same number (rounded up) for every split
    const int g_first = first >> 4, g_last = pos >> 4;
    const int per = (g_last - g_first + n_splits) / n_splits;
    const int g0 = g_first + split * per;
    const int g1 = min(g_last, g0 + per - 1);
    const int key_lo = max(first, g0 << 4), key_hi = min(pos, (g1 << 4) + 15);
    const int c = lane & 3, r = lane >> 2;

    DAcc<HD, NT> acc;
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) acc.o[tt][i][0] = acc.o[tt][i][1] = acc.o[tt][i][2] = acc.o[tt][i][3] = 0.0f;
        acc.m[tt][0] = acc.m[tt][1] = -INFINITY;
        acc.l[tt][0] = acc.l[tt][1] = 0.0f;
    }
    if (g0 + warp <= g1) {
        // the query of head (8 * tt + r) as the right-hand operand of the first product
        uint4 qf[NT][HD / 32];
        const __nv_bfloat16* qbase = q + out_row;
#pragma unroll
        for (int tt = 0; tt < NT; ++tt)
#pragma unroll
            for (int j = 0; j < HD / 32; ++j)
                qf[tt][j] = 8 * tt + r < G ? ld16(qbase + (size_t)(8 * tt + r) * HD + (c + 4 * j) * 8)
                                           : make_uint4(0, 0, 0, 0);
        Pages pg{k_pages, v_pages, block_table + (size_t)seq * bt_stride, n_kv, kvh};
        int gi = g0 + warp;
        DGroup<HD> cur, nxt;
        d_load_group<HD>(cur, pg, gi << 4, key_lo, key_hi, lane);
        while (true) {
            const int gn = gi + 4;
            const bool more = gn <= g1;
            if (more) d_load_group<HD>(nxt, pg, gn << 4, key_lo, key_hi, lane);
            d_consume_group<HD, NT>(acc, qf, cur, gi << 4, key_lo, key_hi, scale2, lane);
            if (!more) break;
            cur = nxt;
            gi = gn;
        }
    }
    // the lanes that share c hold partial sums of the same two heads
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int sh = 4; sh <= 16; sh <<= 1) acc.l[tt][e] += __shfl_xor_sync(0xffffffffu, acc.l[tt][e], sh);
    // the four warps' results meet in shared memory
    constexpr int W = HD + 2;
    float* mine = sm + (size_t)warp * G * W;
#pragma unroll
    for (int tt = 0; tt < NT; ++tt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int head = 8 * tt + 2 * c + e;
            if (head < G) {
#pragma unroll
                for (int i = 0; i < HD / 16; ++i) {
                    const int d = (i >> 2) * 64 + r * 8 + (i & 3);
                    mine[head * W + d] = acc.o[tt][i][e];
                    mine[head * W + d + 4] = acc.o[tt][i][2 + e];
                }
                if (r == 0) {
                    mine[head * W + HD] = acc.m[tt][e];
                    mine[head * W + HD + 1] = acc.l[tt][e];
                }
            }
        }
    __syncthreads();
    const size_t pb = ((size_t)t * n_kv + kvh) * n_splits + split;
    for (int i = threadIdx.x; i < G * HD; i += 128) {
        const int head = i / HD, d = i % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, sm[(w * G + head) * W + HD]);
        float o = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm[(w * G + head) * W + HD];
            const float cw = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            o = fmaf(sm[(w * G + head) * W + d], cw, o);
            l = fmaf(sm[(w * G + head) * W + HD + 1], cw, l);
        }
        if (n_splits == 1) {
            out[out_row + i] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
        } else {
            part_o[pb * G * HD + i] = o;
            if (d == 0) {
                part_ml[(pb * G + head) * 2] = m;
                part_ml[(pb * G + head) * 2 + 1] = l;
            }
        }
    }
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

template <int HD>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table, int bt_stride,
                  const int* tok_seq, const int* tok_pos, void* out, float* scratch, int n_tok, int n_heads, int n_kv,
                  float scale, int window, int n_splits, cudaStream_t stream) {
    const int G = n_heads / n_kv;
    const size_t smem = (size_t)4 * G * (HD + 2) * sizeof(float);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_tok * n_kv * n_splits * G * HD : nullptr;
    dim3 grid(n_splits, n_kv, n_tok);
    if (G <= 8)
        decode_kernel<HD, 1><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                                                          (const __nv_bfloat16*)v_pages, block_table, bt_stride,
                                                          tok_seq, tok_pos, (__nv_bfloat16*)out, part_o, part_ml,
                                                          n_heads, n_kv, scale * kLog2e, window);
    else
        decode_kernel<HD, 2><<<grid, 128, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
                                                          (const __nv_bfloat16*)v_pages, block_table, bt_stride,
                                                          tok_seq, tok_pos, (__nv_bfloat16*)out, part_o, part_ml,
                                                          n_heads, n_kv, scale * kLog2e, window);
    NN_LAUNCH_OK("attention decode");
    if (n_splits > 1) {
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
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        configured = true;
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
