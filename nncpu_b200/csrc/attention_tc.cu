// Prefill attention over the paged cache on the 5th-generation tensor cores
// (bfloat16, head size 64 or 128, causal with an optional window).
//
// A block owns 128 consecutive new tokens of one sequence and one or two query
// heads that share a key/value head.  It walks the pages of keys those tokens
// may see, two pages (128 keys) a step:
//   * a producer thread copies the pages' K and V tiles to shared memory by TMA
//     (128-byte swizzle); the K ring and the V ring advance separately, since K
//     is free once the scores are computed and V once O has been updated;
//   * one thread issues tcgen05.mma: S = Q . K^T into the head's columns of
//     tensor memory, and O += P . V with P read from tensor memory (it lies
//     over the second half of S) and V read as an MN-major operand straight
//     from the pages' layout.  The head's next scores follow its O update at
//     once, so the tensor core works for one head while the other head's
//     warpgroup computes exponentials;
//   * a warpgroup per head owns one query row per thread: it reads its row of
//     S from tensor memory, scales and masks it, and stores the weights P
//     as bfloat16 pairs back into tensor memory, keeping sum and maximum in
//     32-bit.  Weights are taken against a reference maximum that lags behind
//     the true one: as long as a step's weights of a row add up to at most
//     2^8 nothing can have overflowed and the reference stays; otherwise the
//     row's largest score is found, the reference moves up to it, the row's O
//     (between two O updates, never under one) and sum are rescaled and the
//     step's weights computed again.
// The output row is O / sum.  The reference computes the same attention row by
// row (crates/nncpu/src/model/forward.rs:141-160,383-426); softmax runs in 32-bit here
// as there.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out sets
// *status, the other roles run into their own limits, copies in flight are
// waited for and the block frees its tensor memory on the common exit.

#include <map>
#include <mutex>
#include <tuple>

#define NN_LIB attention_tc
#define NN_LAUNCH_OVERLAP
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int kQRows = 128;   // query rows per block = tensor-core M
constexpr int kKeys = 2 * kPage;  // keys per step: two cache pages
constexpr int kStages = 2;    // steps of K and of V in flight
constexpr int kStreamCols = 256;  // tensor-memory columns per head: S (P over its second half) | O
constexpr int kPOffset = 64;      // P lies over the second half of S
constexpr float kSumLimit = 256.0f;  // a step's weights of a row may add up to this before the row's reference maximum is moved

enum AttnStatus : int { kTimeoutQ = 201, kTimeoutStage = 202, kTimeoutK = 203, kTimeoutV = 204, kTimeoutS = 205,
                        kTimeoutP = 206, kTimeoutPv = 207 };

struct AttnParams {
    const int* block_table;
    int bt_stride;
    const int* cu_seqlens;
    const int* tok_pos;
    __nv_bfloat16* out;
    int n_seqs, n_heads, n_kv;
    float scale2;   // softmax scale times log2(e)
    int window;
    int* status;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Descriptor of an MN-major operand in 128-byte swizzle: rows of 64 elements (128 bytes) along MN,
// consecutive k 128 bytes apart, groups of 8 k 1024 bytes apart, the next 64 along MN `lbo` bytes on.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// P . V with P taken from tensor memory (the A operand) and V from shared memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Threads: warp 0 producer, warp 1 tensor-core issue and tensor memory, then one warpgroup per head.
template <int HD, int kStreams>
__global__ void __launch_bounds__(64 + 128 * kStreams, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
    constexpr int kSlabs = HD / 64;                 // 64-element (128-byte) column blocks of a head
    constexpr int kQBytes = kQRows * HD * 2;        // one head's query tile
    constexpr int kQSlab = kQRows * 128;
    constexpr int kPageBytes = kPage * HD * 2;      // one page of K or of V for one head
    constexpr int kKvSlab = kKeys * 128;            // a stage holds kKeys rows of 128 bytes per column block
    constexpr int kKvBytes = kSlabs * kKvSlab;      // one stage of K or of V
    constexpr int kTmemCols = kStreams * kStreamCols;
    static_assert(HD == 64 || HD == 128, "head size 64 or 128");
    static_assert(kKeys + HD <= kStreamCols, "S (with P over its second half) and O fit a head's columns");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_q = smem;                                   // [kStreams][kSlabs][128 rows][128 B]
    uint8_t* smem_k = smem_q + kStreams * kQBytes;            // [kStages][kSlabs][128 keys][128 B]
    uint8_t* smem_v = smem_k + kStages * kKvBytes;            // the same
    uint64_t* q_full = (uint64_t*)(smem_v + kStages * kKvBytes);
    uint64_t* k_full = q_full + 1;                            // [kStages]
    uint64_t* v_full = k_full + kStages;                      // [kStages]
    uint64_t* k_empty = v_full + kStages;                     // [kStages]
    uint64_t* v_empty = k_empty + kStages;                    // [kStages]
    uint64_t* s_full = v_empty + kStages;                     // [kStreams]
    uint64_t* p_full = s_full + kStreams;                     // [kStreams]
    uint64_t* o_done = p_full + kStreams;                     // [kStreams]
    uint32_t* tmem_slot = (uint32_t*)(o_done + kStreams);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Launched to start while the kernel before it ends (its set-up needs nothing of that kernel; the step's
    // metadata was copied before the step's first kernel).  It waits before its first copy of q or of a page.
    let_next_kernel_start();

    // the block's 128 query rows: tiles are numbered within each sequence from its end (long spans first)
    int tile = blockIdx.y;
    int seq = -1, q0 = 0, q_end = 0;
    for (int b = 0; b < p.n_seqs; ++b) {
        const int a = p.cu_seqlens[b], e = p.cu_seqlens[b + 1];
        const int n_tiles = (e - a + kQRows - 1) / kQRows;
        if (tile < n_tiles) {
            seq = b;
            q0 = a + (n_tiles - 1 - tile) * kQRows;
            q_end = e;
            break;
        }
        tile -= n_tiles;
    }
    if (seq < 0) return;   // the grid is an upper bound; the whole block leaves before anything is set up
    const int n_rows = min(kQRows, q_end - q0);
    const int pos0 = p.tok_pos[q0];                  // positions of a sequence's new tokens are consecutive
    const int key_hi = pos0 + n_rows - 1;
    const int key_lo = (p.window > 0 && pos0 + 1 > p.window) ? pos0 + 1 - p.window : 0;
    const int page_lo = key_lo / kPage, page_hi = key_hi / kPage;
    const int n_pages = page_hi - page_lo + 1;
    const int n_steps = (n_pages + 1) / 2;           // two pages a step; the last step may hold one
    // the heads of a key/value head are dealt out two to a block; an odd group's last block has one
    const int group = p.n_heads / p.n_kv;
    const int per_kv = (group + kStreams - 1) / kStreams;
    const int kvh = blockIdx.x / per_kv;
    const int head0 = kvh * group + (blockIdx.x % per_kv) * kStreams;
    const int n_streams = min(kStreams, group - (blockIdx.x % per_kv) * kStreams);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int t = 0; t < kStreams; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 128);
            mbar_init(&o_done[t], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    wait_for_previous_kernels();

    if (warp == 0) {
        if (lane == 0) {
            const int* table = p.block_table + (size_t)seq * p.bt_stride;
            mbar_expect_tx(q_full, n_streams * kQBytes);
            for (int t = 0; t < n_streams; ++t)
                for (int s = 0; s < kSlabs; ++s)
                    tma_load_2d(smem_q + t * kQBytes + s * kQSlab, &map_q, q_full, (head0 + t) * HD + 64 * s, q0);
            // K tiles are free again once their scores are computed, V tiles once O has been updated, so the two
            // rings advance on their own: one thread polls both without blocking on either
            int jk = 0, jv = 0;
            bool ok = true;
            unsigned long long t0 = global_ns();
            while (jk < n_steps || jv < n_steps) {
                bool moved = false;
                if (jk < n_steps && mbar_test_wait(&k_empty[jk % kStages], ((jk / kStages) & 1) ^ 1)) {
                    const int st = jk % kStages;
                    const int pages = min(2, n_pages - 2 * jk);
                    mbar_expect_tx(&k_full[st], pages * kPageBytes);
                    for (int pg = 0; pg < pages; ++pg)
                        for (int s = 0; s < kSlabs; ++s)
                            tma_load_4d(smem_k + st * kKvBytes + s * kKvSlab + pg * (kPage * 128), &map_k, &k_full[st],
                                        64 * s, 0, kvh, table[page_lo + 2 * jk + pg]);
                    ++jk;
                    moved = true;
                }
                if (jv < jk && mbar_test_wait(&v_empty[jv % kStages], ((jv / kStages) & 1) ^ 1)) {
                    const int st = jv % kStages;
                    const int pages = min(2, n_pages - 2 * jv);
                    mbar_expect_tx(&v_full[st], pages * kPageBytes);
                    for (int pg = 0; pg < pages; ++pg)
                        for (int s = 0; s < kSlabs; ++s)
                            tma_load_4d(smem_v + st * kKvBytes + s * kKvSlab + pg * (kPage * 128), &map_v, &v_full[st],
                                        64 * s, 0, kvh, table[page_lo + 2 * jv + pg]);
                    ++jv;
                    moved = true;
                }
                if (moved) {
                    t0 = global_ns();
                } else if (global_ns() - t0 > kWaitLimitNs) {
                    atomicExch(p.status, kTimeoutStage);
                    ok = false;
                    break;
                }
            }
            if (!ok) {
                // let the copies in flight land before the block gives up its shared memory
                mbar_wait(q_full, 0);
                for (int r = max(0, jk - kStages); r < jk; ++r) mbar_wait(&k_full[r % kStages], (r / kStages) & 1);
                for (int r = max(0, jv - kStages); r < jv; ++r) mbar_wait(&v_full[r % kStages], (r / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s128 = instr_desc_bf16(kQRows, 128), idesc_s64 = instr_desc_bf16(kQRows, 64);
            constexpr uint32_t idesc_o = instr_desc_bf16(kQRows, HD) | (1u << 16);   // B (V) is MN-major
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(p.status, kTimeoutQ);
            // S_t(i) = Q_t . K(i)^T into the head's S columns; K(i) has landed
            auto issue_scores = [&](int t, int i) {
                const int keys = min(2, n_pages - 2 * i) * kPage;
                const uint32_t k_addr = smem_u32(smem_k + (i % kStages) * kKvBytes);
                const uint32_t q_addr = smem_u32(smem_q + t * kQBytes);
                const uint32_t tmem_s = tmem_base + (uint32_t)(t * kStreamCols);
                const uint32_t idesc = keys == 128 ? idesc_s128 : idesc_s64;
#pragma unroll
                for (int s = 0; s < kSlabs; ++s)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_s, smem_desc_sw128(q_addr + s * kQSlab + k * 32),
                                  smem_desc_sw128(k_addr + s * kKvSlab + k * 32), idesc, (s | k) ? 1u : 0u);
                umma_commit(&s_full[t]);
            };
            if (ok && !mbar_wait(&k_full[0], 0)) {
                atomicExch(p.status, kTimeoutK);
                ok = false;
            }
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int t = 0; t < n_streams; ++t) issue_scores(t, 0);
                umma_commit(&k_empty[0]);
            }
            // Per step and head: O += P . V, then at once the head's next scores (they overwrite P, which the
            // tensor core has read by then: its instructions run in the order they were issued).  While one
            // head's matrices are being multiplied the other head's warpgroup does its exponentials.
            for (int i = 0; i < n_steps && ok; ++i) {
                const int st = i % kStages;
                const int ksteps = min(2, n_pages - 2 * i) * (kPage / 16);
                const bool more = i + 1 < n_steps;
                for (int t = 0; t < n_streams && ok; ++t) {
                    if (!mbar_wait(&p_full[t], i & 1)) {
                        atomicExch(p.status, kTimeoutP);
                        ok = false;
                        break;
                    }
                    if (t == 0) {
                        if (!mbar_wait(&v_full[st], (i / kStages) & 1)) {
                            atomicExch(p.status, kTimeoutV);
                            ok = false;
                            break;
                        }
                        if (more && !mbar_wait(&k_full[(i + 1) % kStages], ((i + 1) / kStages) & 1)) {
                            atomicExch(p.status, kTimeoutK);
                            ok = false;
                            break;
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t v_addr = smem_u32(smem_v + st * kKvBytes);
                    const uint32_t tmem_p = tmem_base + (uint32_t)(t * kStreamCols + kPOffset);
                    const uint32_t tmem_o = tmem_base + (uint32_t)(t * kStreamCols + kKeys);
                    const uint64_t v_desc = smem_desc_sw128_mn(v_addr, kKvSlab);   // 16 keys on: 2048 bytes, 128 in the field
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16_ts(tmem_o, tmem_p + (uint32_t)(k * 8), v_desc + (uint64_t)(k * 128), idesc_o,
                                     (i > 0 || k > 0) ? 1u : 0u);
                    if (ksteps == 8) {
#pragma unroll
                        for (int k = 4; k < 8; ++k)
                            umma_bf16_ts(tmem_o, tmem_p + (uint32_t)(k * 8), v_desc + (uint64_t)(k * 128), idesc_o, 1u);
                    }
                    if (more) issue_scores(t, i + 1);
                    else umma_commit(&o_done[t]);
                }
                if (ok) {
                    umma_commit(&v_empty[st]);
                    if (more) umma_commit(&k_empty[(i + 1) % kStages]);
                }
            }
        }
    } else {
        const int t = (warp - 2) >> 2;            // which head of the block
        const int quarter = warp & 3;             // the tensor-memory lanes this warp may touch
        const int row = quarter * 32 + lane;
        const int h = head0 + t;
        const int lim_hi = row < n_rows ? pos0 + row : -1;
        const int lim_lo = (p.window > 0 && lim_hi + 1 > p.window) ? lim_hi + 1 - p.window : 0;
        const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(t * kStreamCols);
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = t < n_streams;   // the second warpgroup of a block with one head has nothing to do
        for (int i = 0; ok && i < n_steps; ++i) {
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], i & 1));
            if (!ok) {
                if (lane == 0) atomicExch(p.status, kTimeoutS);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int halves = min(2, n_pages - 2 * i);
            const int k_base = (page_lo + 2 * i) * kPage;
            // A step costs one pass over the row's scores: weights against the reference maximum as it stands (as
            // bfloat16 pairs) and their sum.  The largest score is not looked for: a sum of at most 2^8 proves that
            // no weight is above 2^8.  Only when a row's sum says otherwise (or the row has seen no key yet) is the
            // largest score found in a pass of its own; then the reference moves up to it, O and the sum so far
            // follow, and the weights are computed again.  The O update of the step before is complete (these
            // scores were issued after it), so O may be touched.
            float sum = 0.0f;
            uint32_t w[2][32];   // P of the two pages, stored once the reference maximum is settled: P overwrites S
            auto load_half = [&](int hf, uint32_t (&u)[64]) {
                tmem_ld64(tmem_row + (uint32_t)(64 * hf), u);
                const int kb = k_base + 64 * hf;
                if (!(kb >= lim_lo && kb + 63 <= lim_hi)) {
                    // the page crosses this row's limits
#pragma unroll
                    for (int c = 0; c < 64; ++c)
                        if (kb + c < lim_lo || kb + c > lim_hi) u[c] = 0xff800000u;   // -inf
                }
            };
            auto weights = [&]() {
                const float neg_m = m_ref == -INFINITY ? 0.0f : 0.0f - m_ref;
                float sm[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (hf < halves) {
                        uint32_t u[64];
                        load_half(hf, u);
#pragma unroll
                        for (int c = 0; c < 64; c += 2) {
                            const float e0 = fast_exp2(fmaf(__uint_as_float(u[c]), p.scale2, neg_m));
                            const float e1 = fast_exp2(fmaf(__uint_as_float(u[c + 1]), p.scale2, neg_m));
                            sm[c & 3] += e0;
                            sm[(c & 3) + 1] += e1;
                            w[hf][c >> 1] = pack_bf16(e0, e1);
                        }
                    }
                }
                sum = (sm[0] + sm[1]) + (sm[2] + sm[3]);
            };
            const bool unseen = __any_sync(0xffffffffu, m_ref == -INFINITY && lim_hi >= 0);
            if (!unseen) weights();
            if (unseen || __any_sync(0xffffffffu, !(sum <= kSumLimit))) {
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    if (hf < halves) {
                        uint32_t u[64];
                        load_half(hf, u);
#pragma unroll
                        for (int c = 0; c < 64; ++c) mx[c & 3] = fmaxf(mx[c & 3], __uint_as_float(u[c]));
                    }
                }
                const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale2;   // the scale is positive
                float alpha = 1.0f;
                if (tmax > m_ref) {
                    alpha = fast_exp2(m_ref - tmax);    // 0 when nothing was seen yet
                    m_ref = tmax;
                    l *= alpha;
                }
                if (i > 0) {
#pragma unroll 1
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem_row + (uint32_t)(kKeys + c0), o);
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        tmem_st32(tmem_row + (uint32_t)(kKeys + c0), o);
                    }
                }
                weights();
            }
            l += sum;
            tmem_st32(tmem_row + (uint32_t)kPOffset, w[0]);
            if (halves == 2) tmem_st32(tmem_row + (uint32_t)(kPOffset + 32), w[1]);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&p_full[t]);
        }
        if (ok) {
            ok = __all_sync(0xffffffffu, mbar_wait(&o_done[t], 0));
            if (!ok && lane == 0) atomicExch(p.status, kTimeoutPv);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = p.out + (size_t)(q0 + row) * ((size_t)p.n_heads * HD) + (size_t)h * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_row + (uint32_t)(kKeys + c0), o);
                if (row < n_rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = w;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps (cached by what they describe) and the launcher.
// ---------------------------------------------------------------------------
struct MapCache {
    std::mutex lock;
    std::map<std::tuple<const void*, long, long, long, int>, CUtensorMap> maps;

    // kind 0: queries [rows, cols] in boxes of 128 rows x 64; kind 1: pages [n_pages, n_kv, 64, hd] in boxes of
    // one head's 64 keys x 64
    int get(CUtensorMap* out, const void* base, long d0, long d1, long d2, int kind) {
        std::lock_guard<std::mutex> g(lock);
        const auto key = std::make_tuple(base, d0, d1, d2, kind);
        auto it = maps.find(key);
        if (it == maps.end()) {
            EncodeTiledFn fn = encode_tiled();
            NN_CHECK(fn != nullptr, "attention (tensor cores): the driver does not offer cuTensorMapEncodeTiled");
            CUtensorMap m;
            CUresult r;
            if (kind == 0) {
                const cuuint64_t dims[2] = {(cuuint64_t)d1, (cuuint64_t)d0};
                const cuuint64_t strides[1] = {(cuuint64_t)d1 * 2};
                const cuuint32_t box[2] = {64, (cuuint32_t)kQRows};
                const cuuint32_t elem[2] = {1, 1};
                r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            } else {
                const long n_pages = d0, n_kv = d1, hd = d2;
                const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)kPage, (cuuint64_t)n_kv, (cuuint64_t)n_pages};
                const cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)hd * 2 * kPage,
                                               (cuuint64_t)hd * 2 * kPage * n_kv};
                const cuuint32_t box[4] = {64, (cuuint32_t)kPage, 1, 1};
                const cuuint32_t elem[4] = {1, 1, 1, 1};
                r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            }
            NN_CHECK(r == CUDA_SUCCESS,
                     "attention (tensor cores): cuTensorMapEncodeTiled failed with code %d (kind %d, %ld x %ld x %ld)",
                     (int)r, kind, d0, d1, d2);
            if (maps.size() > 65536) maps.clear();
            it = maps.emplace(key, m).first;
        }
        *out = it->second;
        return 0;
    }
};

MapCache g_maps;

template <int HD, int kStreams>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnParams& p, int n_tok,
           cudaStream_t stream) {
    constexpr int smem = kStreams * kQRows * HD * 2 + 2 * kStages * kKeys * HD * 2 + 256 + 1024;
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<HD, kStreams>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        NN_CHECK(e == cudaSuccess, "attention (tensor cores): %d bytes of shared memory refused: %s", smem,
                 cudaGetErrorString(e));
    }
    // tiles: an upper bound, since the sequence boundaries live on the device; spare blocks leave at once
    const int group = p.n_heads / p.n_kv;
    const dim3 grid(p.n_kv * ((group + kStreams - 1) / kStreams), (n_tok + kQRows - 1) / kQRows + p.n_seqs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(64 + 128 * kStreams);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = overlap_attribute(attr);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_tc_kernel<HD, kStreams>, mq, mk, mv, p);
    NN_CHECK(e == cudaSuccess, "attention prefill (tensor cores): launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

extern "C" int nncpu_attention_prefill_tc_supported(int n_heads, int n_kv, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_heads > 0 && n_heads % n_kv == 0;
}

// q and out: bfloat16 [n_tok, n_heads * head_dim]; K and V pages: bfloat16 [n_pages, n_kv, 64, head_dim] holding
// every key the new tokens may see, their own included; cu_seqlens [n_seqs + 1] row ranges of the sequences;
// tok_pos [n_tok] positions (consecutive within a sequence).  *status receives a code if a wait runs out.
extern "C" int nncpu_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, int n_pages,
                                          const int* block_table, int bt_stride, const int* cu_seqlens,
                                          const int* tok_pos, void* out, int n_tok, int n_seqs, int n_heads, int n_kv,
                                          int head_dim, float scale, int window, int* status, void* stream_) {
    NN_CHECK(nncpu_attention_prefill_tc_supported(n_heads, n_kv, head_dim),
             "attention (tensor cores): head size %d with %d heads over %d key/value heads is not supported "
             "(head size 64 or 128, heads a multiple of key/value heads)", head_dim, n_heads, n_kv);
    NN_CHECK(n_tok >= 0 && n_seqs >= 0 && window >= 0 && n_pages > 0, "attention (tensor cores): %d tokens of %d sequences, %d pages",
             n_tok, n_seqs, n_pages);
    NN_CHECK(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0 &&
             ((uintptr_t)out % 16) == 0, "attention (tensor cores): operands must be 16-byte aligned");
    NN_CHECK(status != nullptr, "attention (tensor cores): no status word");
    if (n_tok == 0 || n_seqs == 0) return 0;
    CUtensorMap mq, mk, mv;
    if (int e = g_maps.get(&mq, q, n_tok, (long)n_heads * head_dim, 0, 0)) return e;
    if (int e = g_maps.get(&mk, k_pages, n_pages, n_kv, head_dim, 1)) return e;
    if (int e = g_maps.get(&mv, v_pages, n_pages, n_kv, head_dim, 1)) return e;
    AttnParams p;
    p.block_table = block_table;
    p.bt_stride = bt_stride;
    p.cu_seqlens = cu_seqlens;
    p.tok_pos = tok_pos;
    p.out = (__nv_bfloat16*)out;
    p.n_seqs = n_seqs;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.scale2 = scale * 1.4426950408889634f;
    p.window = window;
    p.status = status;
    cudaStream_t stream = (cudaStream_t)stream_;
    // two heads to a block where a key/value head has two to give; one head per block otherwise
    if (n_heads == n_kv)
        return head_dim == 64 ? launch<64, 1>(mq, mk, mv, p, n_tok, stream) : launch<128, 1>(mq, mk, mv, p, n_tok, stream);
    return head_dim == 64 ? launch<64, 2>(mq, mk, mv, p, n_tok, stream) : launch<128, 2>(mq, mk, mv, p, n_tok, stream);
}
