// bfloat16 matrix product for sm_100a on the 5th-generation tensor cores:
//   C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias[N])
// or, with the gated-activation epilogue, C[M, N/2] = silu(gate) * up where the
// rows of W hold gate and up rows interleaved in blocks of 8.
//
// Operand tiles come to shared memory by TMA (128-byte swizzle); one elected
// thread issues tcgen05.mma with the accumulator in tensor memory; four warps
// read the accumulator back with tcgen05.ld for the epilogue.  The kernels are
// persistent: each block walks a list of work items and keeps two accumulators
// in tensor memory, so the epilogue of one item runs under the matrix
// instructions of the next.
//
// The tensor-core M operand is always a 128-row tile of "A" and the N operand a
// BN-row tile of "B":
//   * many tokens:  A = activations, B = weights; from 512 tokens on two SMs
//     share a 256 x 256 tile (gemm_pair_kernel);
//   * few tokens (up to 256):  A = weights, B = activations, and the epilogue
//     stores the tile transposed: every weight byte is read once and no
//     tensor-core row is spent on padding.  There are few output tiles then, so
//     K is cut: either the k-blocks of all tiles are dealt out evenly to the
//     blocks and a second kernel adds the parts of split tiles
//     (gemm_streamk_kernel), or a thread-block cluster shares a tile and adds
//     its slices through distributed shared memory (gemm_cluster_kernel).
//     Both add in a fixed order: the sum does not depend on timing, and no
//     block waits for another outside a cluster barrier.
// The reference computes the same products with its own BF16 row kernels
// (crates/nncpu/src/kernels/mod.rs:454-485, crates/nncpu/src/kernels/scalar.rs:555-567);
// accumulation is 32-bit here as there.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out sets
// *status and the block leaves through the common exit, which frees its
// tensor memory.

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#define NN_LIB gemm_sm100
#define NN_LAUNCH_OVERLAP
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int kBlockM = 128;  // rows of the A tile = tensor-core M
constexpr int kBlockK = 64;   // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;    // K of one tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;  // warp 0: TMA, warp 1: MMA and tensor memory, warps 2-5: epilogue
// The kernel for pairs of SMs has eight epilogue warps: two per quarter of the tensor-memory lanes, each with one
// half of a tile's 256 columns, so that an epilogue that no product hides (the last tile's) takes half as long.
constexpr int kPairThreads = 64 + 256;

enum GemmStatus : int { kOk = 0, kTimeoutEmpty = 101, kTimeoutFull = 102, kTimeoutAccumFull = 103,
                        kTimeoutAccumEmpty = 104 };
enum Epilogue : int { kPlain = 0, kSwiglu = 1, kQkv = 2 };

__device__ __forceinline__ float silu_mul(float g, float u) { return (g * (1.0f / (1.0f + expf(0.0f - g)))) * u; }

// What the fused q/k/v epilogue needs: the output columns are heads of 128 (queries, then keys, then values).
struct QkvParams {
    __nv_bfloat16* q_out;      // [tokens, n_heads * 128]
    __nv_bfloat16* k_pages;    // [pages, n_kv, 64, 128]
    __nv_bfloat16* v_pages;
    const void* q_gamma;       // per-head norm weights, or null
    const void* k_gamma;
    int g_dt;
    float eps;
    const float2* cos_sin;     // [64, tokens] (cos, sin) of pair i at each token's position, or null
    const int* tok_seq;        // the cache slot of each token (-1: none)
    const int* tok_pos;
    const int* block_table;
    int bt_stride;
    int n_heads, n_kv;
};

struct GemmParams {
    int rows_a, rows_b, K;
    int tiles_a, tiles_b, splits, kb_total;
    void* out;         // [tokens, ldc]
    const void* bias;  // per output feature, or null
    int out_dt, bias_dt;
    int ldc;
    int accumulate;  // add to what `out` holds
    int swap;        // 0: A rows are tokens; 1: A rows are output features
    int vec;         // rows of `out` may be written 16 bytes at a time
    float* scratch;  // partial tiles of products that deal k-blocks out evenly: two slots of [BN][128] floats per block
    int* status;
    unsigned long long wait_ns;  // limit of every mbarrier wait of gemm_bf16_kernel; 0: the default (2 s)
    int tx_extra;      // bytes added to what a stage's barrier expects (the wait probe only: they never arrive)
    QkvParams qkv;     // epilogue kQkv only
    NormFusion nf;     // pairs of SMs only: the norms that ride on this product (common.cuh)
};

// Stores up to 16 accumulator values of one thread: A row `a_row`, B rows b0 .. b0 + ncols - 1
// (ncols below 16 only when A rows are output features).
template <int kEpi>
__device__ __forceinline__ void store16(const GemmParams& p, int a_row, int b0, float (&v)[16], int ncols = 16) {
    const bool a_ok = a_row < p.rows_a;
    if (kEpi == kSwiglu) {
        if (!p.swap) {
            // columns hold 8 gate values, then the 8 up values of the same outputs
            if (!a_ok || b0 >= p.rows_b) return;
            const size_t o = (size_t)a_row * p.ldc + (b0 >> 1);
            float act[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) act[j] = silu_mul(v[j], v[j + 8]);
            if (p.vec && p.out_dt == DT_BF16) {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(act[2 * j], act[2 * j + 1]);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = *reinterpret_cast<uint4*>(h);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) st_f(p.out, o + j, p.out_dt, act[j]);
            }
        } else {
            // Rows hold 8 gate rows, then 8 up rows: lane l and lane l ^ 8 hold the gate and the up value of one
            // feature.  The pair shares the work: of two neighbouring tokens the gate lane finishes the first and
            // the up lane the second, so every lane computes one activation per two columns.
            const bool is_gate = (a_row & 8) == 0;
            const int feature = (a_row >> 4) * 8 + (a_row & 7);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                const float o0 = __shfl_xor_sync(0xffffffffu, v[j], 8);
                const float o1 = __shfl_xor_sync(0xffffffffu, v[j + 1], 8);
                const float g = is_gate ? v[j] : o1, u = is_gate ? o0 : v[j + 1];
                const int jj = is_gate ? j : j + 1;
                const int tok = b0 + jj;
                if (a_ok && jj < ncols && tok < p.rows_b)
                    st_f(p.out, (size_t)tok * p.ldc + feature, p.out_dt, silu_mul(g, u));
            }
        }
        return;
    }
    if (!a_ok) return;
    if (!p.swap) {
        const size_t o = (size_t)a_row * p.ldc + b0;
        if (p.vec && b0 + 16 <= p.rows_b) {
            if (p.bias) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += ld_f(p.bias, b0 + j, p.bias_dt);
            }
            if (p.out_dt == DT_F32) {
                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o);
                if (p.accumulate) {
                    // all four loads before the first store: one round trip instead of four
                    float4 y[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) y[j] = dst[j];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[4 * j] += y[j].x; v[4 * j + 1] += y[j].y; v[4 * j + 2] += y[j].z; v[4 * j + 3] += y[j].w;
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    __nv_bfloat162 h[4];
                    if (p.accumulate) {
                        const uint4 y = *reinterpret_cast<const uint4*>(dst + 8 * half);
                        const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __bfloat1622float2(yh[j]);
                            h[j] = __floats2bfloat162_rn(v[8 * half + 2 * j] + f.x, v[8 * half + 2 * j + 1] + f.y);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            h[j] = __floats2bfloat162_rn(v[8 * half + 2 * j], v[8 * half + 2 * j + 1]);
                    }
                    *reinterpret_cast<uint4*>(dst + 8 * half) = *reinterpret_cast<uint4*>(h);
                }
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int col = b0 + j;
            if (col >= p.rows_b) break;
            float x = v[j];
            if (p.bias) x += ld_f(p.bias, col, p.bias_dt);
            if (p.accumulate) x += ld_f(p.out, o + j, p.out_dt);
            st_f(p.out, o + j, p.out_dt, x);
        }
    } else {
        // C[b0 + j, a_row]: the lanes of a warp write neighbouring elements.  What is already there is loaded
        // for all 16 before the first store, so the loads are in flight together.
        const float b = p.bias ? ld_f(p.bias, a_row, p.bias_dt) : 0.0f;
        float old[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = b0 + j;
            old[j] = (p.accumulate && tok < p.rows_b && j < ncols) ? ld_f(p.out, (size_t)tok * p.ldc + a_row, p.out_dt) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = b0 + j;
            if (tok >= p.rows_b || j >= ncols) break;
            st_f(p.out, (size_t)tok * p.ldc + a_row, p.out_dt, (v[j] + b) + old[j]);
        }
    }
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

template <int BN, int kStages, int kEpi>
__global__ void __launch_bounds__(kThreads)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
    constexpr int kBytesA = kBlockM * kBlockK * 2;
    constexpr int kBytesB = BN * kBlockK * 2;
    constexpr int kAccCols = BN < 32 ? 32 : BN;   // columns of one accumulator
    constexpr int kTmemCols = 2 * kAccCols;       // two accumulators; a power of two >= 64
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kBytesA;
    uint64_t* full = (uint64_t*)(smem_b + kStages * kBytesB);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;   // [2]
    uint64_t* acc_empty = acc_full + 2;     // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.tiles_a * p.tiles_b;
    const unsigned long long limit = p.wait_ns ? p.wait_ns : kWaitLimitNs;
    // This block's k-blocks in the order it works through them: run r is k-block r % kb_total of its tile r / kb_total.
    const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int my_runs = my_tiles * p.kb_total;
    const int n_first = min(kStages, my_runs);   // copies that need no free stage

    let_next_kernel_start();
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // The first weights are asked for before anything that the kernel before this one may still be writing is
        // touched (with swapped operands the weights are A).
        for (int r = 0; r < n_first; ++r) {
            const int w = blockIdx.x + (r / p.kb_total) * gridDim.x, kb = r % p.kb_total;
            mbar_expect_tx(&full[r], kBytesA + kBytesB + p.tx_extra);
            if (p.swap) tma_load_2d(smem_a + r * kBytesA, &map_a, &full[r], kb * kBlockK, (w % p.tiles_a) * kBlockM);
            else tma_load_2d(smem_b + r * kBytesB, &map_b, &full[r], kb * kBlockK, (w / p.tiles_a) * BN);
        }
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

    // Work item w: output tile (w % tiles_a, w / tiles_a), all of K.
    if (warp == 0) {
        if (lane == 0) {
            int issued = n_first;
            bool ok = true;
            for (int r = 0; r < n_first; ++r) {   // the activations of the first copies
                const int w = blockIdx.x + (r / p.kb_total) * gridDim.x, kb = r % p.kb_total;
                if (p.swap) tma_load_2d(smem_b + r * kBytesB, &map_b, &full[r], kb * kBlockK, (w / p.tiles_a) * BN);
                else tma_load_2d(smem_a + r * kBytesA, &map_a, &full[r], kb * kBlockK, (w % p.tiles_a) * kBlockM);
            }
            for (int r = n_first; r < my_runs; ++r) {
                const int w = blockIdx.x + (r / p.kb_total) * gridDim.x, kb = r % p.kb_total;
                const int m0 = (w % p.tiles_a) * kBlockM, n0 = (w / p.tiles_a) * BN;
                const int s = r % kStages;
                if (!mbar_wait(&empty[s], ((r / kStages) & 1) ^ 1, limit)) {
                    atomicExch(p.status, kTimeoutEmpty);
                    ok = false;
                    break;
                }
                mbar_expect_tx(&full[s], kBytesA + kBytesB + p.tx_extra);
                tma_load_2d(smem_a + s * kBytesA, &map_a, &full[s], kb * kBlockK, m0);
                tma_load_2d(smem_b + s * kBytesB, &map_b, &full[s], kb * kBlockK, n0);
                issued = r + 1;
            }
            if (!ok) {
                // let the copies already in flight land before the block gives up its shared memory
                for (int r = max(0, issued - kStages); r < issued; ++r) mbar_wait(&full[r % kStages], (r / kStages) & 1, limit);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kBlockM, BN);
            int kb_run = 0, it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_tiles && ok; w += gridDim.x, ++it) {
                const int buf = it & 1;
                if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, limit)) {
                    atomicExch(p.status, kTimeoutAccumEmpty);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kAccCols);
                for (int kb = 0; kb < p.kb_total; ++kb, ++kb_run) {
                    const int s = kb_run % kStages;
                    if (!mbar_wait(&full[s], (kb_run / kStages) & 1, limit)) {
                        atomicExch(p.status, kTimeoutFull);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem_a + s * kBytesA);
                    const uint32_t b_addr = smem_u32(smem_b + s * kBytesB);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                        const uint64_t a_desc = smem_desc_sw128(a_addr + k * kUmmaK * 2);
                        const uint64_t b_desc = smem_desc_sw128(b_addr + k * kUmmaK * 2);
                        umma_bf16(tmem_d, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // Epilogue: warp w may read the tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        // The norm before this product rides on it (swapped operands: tokens are the columns, and all of them are
        // in every tile): the tokens' scales, worked out once by the four epilogue warps while the first tile's
        // products run.
        __shared__ float s_scale[BN];
        const bool scaled = p.nf.bins_in != nullptr;
        if (scaled) {
            for (int j = threadIdx.x - 64; j < BN; j += 128)
                s_scale[j] = j < p.rows_b ? 1.0f / sqrtf(bins_total(p.nf.bins_in + (size_t)j * kBinWords) * (1.0f / (float)p.K) + p.nf.eps)
                                          : 0.0f;
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        int it = 0;
        for (int w = blockIdx.x; w < n_tiles; w += gridDim.x, ++it) {
            const int m0 = (w % p.tiles_a) * kBlockM, n0 = (w / p.tiles_a) * BN;
            const int a_row = m0 + row_in_tile;
            const int buf = it & 1;
            if (!mbar_wait(&acc_full[buf], (it >> 1) & 1, limit)) {
                if (lane == 0) atomicExch(p.status, kTimeoutAccumFull);
                break;
            }
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kAccCols);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                tmem_ld16(taddr + (uint32_t)c0, v);
                if (scaled) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= s_scale[c0 + j];
                }
                store16<kEpi>(p, a_row, n0 + c0, v);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
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
// The same product with the work cut evenly instead of tile by tile ("stream-K"):
// the units are (output tile, k-block) pairs in tile order, and block c of G
// takes the units [c U / G, (c + 1) U / G).  Every block therefore streams the
// same number of weight bytes through one deep pipeline, whatever the number
// of tiles; a tile whose k-blocks fall to several blocks is put together from
// their partial tiles: each block writes its own to scratch memory, and a
// second, wide kernel adds a tile's parts in block order (the order of k) and
// runs the epilogue.  No block waits for another, and the sum does
// not depend on timing.  Used for 65 to 256 tokens (from 17 on where the plan
// asks for it; weights are the 128-row operand), where tiles are few and K is
// long.
// ---------------------------------------------------------------------------
struct Segment {
    int tile, kb0, len;
};

// The first unit of block c.
__device__ __forceinline__ long streamk_start(int c, long units, int blocks) { return (long)c * units / blocks; }

// The block whose range holds unit u.
__device__ __forceinline__ int streamk_owner(long u, long units, int blocks) {
    int c = (int)(u * blocks / units);
    if (c >= blocks) c = blocks - 1;
    while (c + 1 < blocks && streamk_start(c + 1, units, blocks) <= u) ++c;
    while (c > 0 && streamk_start(c, units, blocks) > u) --c;
    return c;
}

// kTM: tiles of 128 A rows that a unit holds.  With two, a k-block of B is copied to shared memory once for 256 rows
// of A: where B (the tokens, with swapped operands) is as large as a tile of A, the copies into shared memory are
// what a block waits for, and a quarter of them goes away.
template <int BN, int kStages, int kEpi, int kTM>
__global__ void __launch_bounds__(kThreads, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    constexpr int kBytesA1 = kBlockM * kBlockK * 2;
    constexpr int kBytesA = kTM * kBytesA1;
    constexpr int kBytesB = BN * kBlockK * 2;
    constexpr int kTileCols = BN < 32 ? 32 : BN;
    constexpr int kAccCols = kTM * kTileCols;
    constexpr int kAccBufs = 2 * kAccCols <= 512 ? 2 : 1;   // two accumulators where tensor memory has room for them
    constexpr int kTmemCols = kAccBufs * kAccCols;
    static_assert(kTmemCols <= 512, "the accumulators fit tensor memory");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kBytesA;
    uint64_t* full = (uint64_t*)(smem_b + kStages * kBytesB);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;   // [2]
    uint64_t* acc_empty = acc_full + 2;     // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.tiles_a * p.tiles_b;
    const long units = (long)n_tiles * p.kb_total;
    const int blocks = (int)gridDim.x;
    let_next_kernel_start();   // the set-up below runs while the kernel before this one ends
    const long u_begin = streamk_start((int)blockIdx.x, units, blocks);
    const long u_end = streamk_start((int)blockIdx.x + 1, units, blocks);
    // this block's next segment from unit u on
    auto segment_at = [&](long u) {
        Segment s;
        s.tile = (int)(u / p.kb_total);
        s.kb0 = (int)(u % p.kb_total);
        const long left = u_end - u;
        s.len = (long)(p.kb_total - s.kb0) < left ? p.kb_total - s.kb0 : (int)left;
        return s;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
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
            int kb_run = 0, issued = 0;
            bool ok = true;
            for (long u = u_begin; u < u_end && ok;) {
                const Segment sg = segment_at(u);
                const int m0 = (sg.tile % p.tiles_a) * (kTM * kBlockM), n0 = (sg.tile / p.tiles_a) * BN;
                for (int kb = sg.kb0; kb < sg.kb0 + sg.len; ++kb, ++kb_run) {
                    const int s = kb_run % kStages;
                    if (!mbar_wait(&empty[s], ((kb_run / kStages) & 1) ^ 1)) {
                        atomicExch(p.status, kTimeoutEmpty);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], kBytesA + kBytesB);
                    // (rows past the end of A are filled with zeros and counted like the others)
#pragma unroll
                    for (int sub = 0; sub < kTM; ++sub)
                        tma_load_2d(smem_a + s * kBytesA + sub * kBytesA1, &map_a, &full[s], kb * kBlockK,
                                    m0 + sub * kBlockM);
                    tma_load_2d(smem_b + s * kBytesB, &map_b, &full[s], kb * kBlockK, n0);
                    issued = kb_run + 1;
                }
                u += sg.len;
            }
            if (!ok) {
                // let the copies already in flight land before the block gives up its shared memory
                for (int r = max(0, issued - kStages); r < issued; ++r) mbar_wait(&full[r % kStages], (r / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kBlockM, BN);
            int kb_run = 0, it = 0;
            bool ok = true;
            for (long u = u_begin; u < u_end && ok; ++it) {
                const Segment sg = segment_at(u);
                const int buf = it % kAccBufs;
                if (!mbar_wait(&acc_empty[buf], ((it / kAccBufs) & 1) ^ 1)) {
                    atomicExch(p.status, kTimeoutAccumEmpty);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kAccCols);
                for (int kb = sg.kb0; kb < sg.kb0 + sg.len; ++kb, ++kb_run) {
                    const int s = kb_run % kStages;
                    if (!mbar_wait(&full[s], (kb_run / kStages) & 1)) {
                        atomicExch(p.status, kTimeoutFull);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem_a + s * kBytesA);
                    const uint32_t b_addr = smem_u32(smem_b + s * kBytesB);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k)
#pragma unroll
                        for (int sub = 0; sub < kTM; ++sub)
                            umma_bf16(tmem_d + (uint32_t)(sub * kTileCols),
                                      smem_desc_sw128(a_addr + sub * kBytesA1 + k * kUmmaK * 2),
                                      smem_desc_sw128(b_addr + k * kUmmaK * 2), idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);
                }
                if (ok) umma_commit(&acc_full[buf]);
                u += sg.len;
            }
        }
    } else {
        // Epilogue: warp w may read the tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        int it = 0;
        for (long u = u_begin; u < u_end; ++it) {
            const Segment sg = segment_at(u);
            u += sg.len;
            const int m0 = (sg.tile % p.tiles_a) * (kTM * kBlockM), n0 = (sg.tile / p.tiles_a) * BN;
            const int buf = it % kAccBufs;
            const bool ok = mbar_wait(&acc_full[buf], (it / kAccBufs) & 1);
            if (!ok && lane == 0) atomicExch(p.status, kTimeoutAccumFull);
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kAccCols);
            if (sg.len == p.kb_total) {
                // the whole tile is this block's
                if (!ok) break;
#pragma unroll 1
                for (int sub = 0; sub < kTM; ++sub) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        float v[16];
                        tmem_ld16(taddr + (uint32_t)(sub * kTileCols + c0), v);
                        store16<kEpi>(p, m0 + sub * kBlockM + row_in_tile, n0 + c0, v);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                continue;
            }
            // A part of the tile: to this block's scratch slot (0: the segment starts inside the tile, which only a
            // block's first segment does; 1: it starts with the tile), column by column so that a warp writes
            // 128 contiguous bytes.  The kernel that follows puts the tile together.
            if (!ok) break;
            float* mine = p.scratch + ((size_t)blockIdx.x * 2 + (sg.kb0 > 0 ? 0 : 1)) * ((size_t)kTM * BN * kBlockM);
#pragma unroll 1
            for (int sub = 0; sub < kTM; ++sub) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr + (uint32_t)(sub * kTileCols + c0), v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[(sub * BN + c0 + j) * kBlockM + row_in_tile] = v[j];
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
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

// Puts together the tiles that gemm_streamk_kernel left in parts: block (tile, 16 columns), thread = row of the
// tile.  The parts of a tile are added in block order, which is the order of k, with all loads in flight at
// once; then the same epilogue as everywhere.  `blocks` is the grid the product ran with.
template <int BN, int kEpi, int kTM>
__global__ void __launch_bounds__(kBlockM)
gemm_streamk_fixup_kernel(const GemmParams p, int blocks) {
    const int tile = blockIdx.x, sub = blockIdx.z, c0 = sub * BN + blockIdx.y * 16;   // c0: the column within a slot
    // launched to start under the end of the product, whose parts it may read only once that kernel is complete
    let_next_kernel_start();
    const long units = (long)p.tiles_a * p.tiles_b * p.kb_total;
    const long t_begin = (long)tile * p.kb_total;
    const int c_first = streamk_owner(t_begin, units, blocks);
    const int c_last = streamk_owner(t_begin + p.kb_total - 1, units, blocks);
    if (c_first == c_last) return;   // one block had the whole tile and stored it
    const int row_in_tile = threadIdx.x;
    const int m0 = (tile % p.tiles_a) * (kTM * kBlockM) + sub * kBlockM, n0 = (tile / p.tiles_a) * BN;
    const size_t slot_floats = (size_t)kTM * BN * kBlockM;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
    wait_for_previous_kernels();
    int c = c_first;
    for (; c + 1 <= c_last; c += 2) {
        const int s0 = streamk_start(c, units, blocks) > t_begin ? 0 : 1;
        const float* a = p.scratch + ((size_t)c * 2 + s0) * slot_floats + c0 * kBlockM + row_in_tile;
        const float* b = p.scratch + ((size_t)(c + 1) * 2 + 0) * slot_floats + c0 * kBlockM + row_in_tile;   // begins inside the tile
        float x[16], y[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            x[j] = __ldcg(a + j * kBlockM);
            y[j] = __ldcg(b + j * kBlockM);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = (v[j] + x[j]) + y[j];
    }
    if (c <= c_last) {
        const int s0 = streamk_start(c, units, blocks) > t_begin ? 0 : 1;
        const float* a = p.scratch + ((size_t)c * 2 + s0) * slot_floats + c0 * kBlockM + row_in_tile;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += __ldcg(a + j * kBlockM);
    }
    store16<kEpi>(p, m0 + row_in_tile, n0 + (int)blockIdx.y * 16, v);
}

// ---------------------------------------------------------------------------
// Few output tiles, many SMs: a thread-block cluster shares one output tile.
// Each block of the cluster multiplies its own slice of K into tensor memory,
// copies the partial tile to its shared memory, and after a cluster barrier
// every block adds up one share of the tile's columns, reading the other
// blocks' partial tiles through distributed shared memory in rank order.  No
// global scratch, and the sum does not depend on timing.
// Used when A rows are output features (few tokens); one tile per cluster.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// Copies `bytes` of this block's shared memory into the shared memory of block `rank` of the cluster; the bytes
// are counted by the mbarrier at `bar_local_addr` in that block.  The copy runs on its own: nothing waits here.
__device__ __forceinline__ void bulk_copy_to_rank(uint32_t dst_local_addr, uint32_t src_addr, uint32_t bytes,
                                                  uint32_t bar_local_addr, uint32_t rank) {
    uint32_t dst, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(dst_local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(bar_local_addr), "r"(rank));
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "r"(src_addr), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared memory of the cluster kernel: the stage ring (which holds the block's partial tile once its products are
// done), then the buffer that receives the cluster's partial sums for this block's share of the tile's columns
// (one slot per sending block), then the barriers.
template <int BN, int kStages>
constexpr size_t cluster_smem_bytes() {
    // shares of BN columns among up to 8 blocks are at most BN / S + 1 wide: S slots of that width fit BN + 8 columns
    return 1024 + (size_t)kStages * (kBlockM * kBlockK * 2 + BN * kBlockK * 2) + (size_t)(BN + 8) * kBlockM * 4 +
           (2 * kStages + 4) * sizeof(uint64_t) + 16;
}

// A cluster of S blocks shares one output tile: block r multiplies the r-th slice of K and owns the r-th share of
// the tile's columns.  When its slice is done a block writes its partial tile into its own shared memory and
// sends every owner its columns with one asynchronous bulk copy each; an owner's mbarrier counts the bytes that
// arrive, and when all S senders' columns are there the owner adds them in sender order and runs the epilogue.
// Nothing is read from another block's memory.  The cluster meets twice off the critical path: once before the
// first copy (every block's shared memory and barrier exist) and once before leaving (every copy out of this
// block's memory has landed, since every owner has seen all of its bytes).
template <int BN, int kStages, int kEpi>
__global__ void __launch_bounds__(kThreads)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    constexpr int kBytesA = kBlockM * kBlockK * 2;
    constexpr int kBytesB = BN * kBlockK * 2;
    constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static_assert(kStages * (kBytesA + kBytesB) >= BN * kBlockM * 4, "the partial tile reuses the stage memory");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kBytesA;
    float* send = (float*)smem;                           // [column][128 rows], after the last tensor-core read of the stages
    float* recv = (float*)(smem_b + kStages * kBytesB);   // [sender][column of mine][128 rows]: at most BN + 8 columns
    uint64_t* full = (uint64_t*)(recv + (BN + 8) * kBlockM);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* arrived = acc_full + 1;                     // counts the bytes of the partial sums sent to this block
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.splits;                     // blocks per cluster
    const int rank = (int)cluster_rank();
    const int tile = blockIdx.x / S;
    const int m0 = (tile % p.tiles_a) * kBlockM, n0 = (tile / p.tiles_a) * BN;
    const int kb0 = (int)((long long)rank * p.kb_total / S), kb1 = (int)((long long)(rank + 1) * p.kb_total / S);
    // columns of the tile that block r owns: [r * BN / S, (r + 1) * BN / S)
    const int c_begin = rank * BN / S, c_end = (rank + 1) * BN / S;
    const int cols = c_end - c_begin;
    const int n_first = min(kStages, kb1 - kb0);   // copies that need no free stage: issued before anything else

    let_next_kernel_start();
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(arrived, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // S senders bring this block's columns, 128 rows of floats each
        mbar_expect_tx(arrived, (uint32_t)(S * cols * kBlockM * 4));
        // the first round of copies starts now, under the set-up of tensor memory and, for the weights, under the end
        // of the kernel before this one (with swapped operands the weights are A)
        for (int i = 0; i < n_first; ++i) {
            mbar_expect_tx(&full[i], kBytesA + kBytesB);
            if (p.swap) tma_load_2d(smem_a + i * kBytesA, &map_a, &full[i], (kb0 + i) * kBlockK, m0);
            else tma_load_2d(smem_b + i * kBytesB, &map_b, &full[i], (kb0 + i) * kBlockK, n0);
        }
        wait_for_previous_kernels();
        for (int i = 0; i < n_first; ++i) {
            if (p.swap) tma_load_2d(smem_b + i * kBytesB, &map_b, &full[i], (kb0 + i) * kBlockK, n0);
            else tma_load_2d(smem_a + i * kBytesA, &map_a, &full[i], (kb0 + i) * kBlockK, m0);
        }
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
    wait_for_previous_kernels();   // thread 0 has waited already; the others read what the product is added to
    // Every block of the cluster has started (its shared memory and its barrier exist) before anyone copies into
    // it.  The wait for this arrival comes just before the copies.  The barriers' initialisation was published by
    // its own fence above, so the arrival orders nothing else and does not flush this thread's memory operations.
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            int issued = n_first;
            bool ok = true;
            for (int kb = kb0 + n_first; kb < kb1; ++kb) {
                const int i = kb - kb0, s = i % kStages;
                if (!mbar_wait(&empty[s], ((i / kStages) & 1) ^ 1)) {
                    atomicExch(p.status, kTimeoutEmpty);
                    ok = false;
                    break;
                }
                mbar_expect_tx(&full[s], kBytesA + kBytesB);
                tma_load_2d(smem_a + s * kBytesA, &map_a, &full[s], kb * kBlockK, m0);
                tma_load_2d(smem_b + s * kBytesB, &map_b, &full[s], kb * kBlockK, n0);
                issued = i + 1;
            }
            if (!ok)
                for (int r = max(0, issued - kStages); r < issued; ++r) mbar_wait(&full[r % kStages], (r / kStages) & 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kBlockM, BN);
            bool ok = true;
            for (int kb = kb0; kb < kb1 && ok; ++kb) {
                const int i = kb - kb0, s = i % kStages;
                if (!mbar_wait(&full[s], (i / kStages) & 1)) {
                    atomicExch(p.status, kTimeoutFull);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem_a + s * kBytesA);
                const uint32_t b_addr = smem_u32(smem_b + s * kBytesB);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k)
                    umma_bf16(tmem_base, smem_desc_sw128(a_addr + k * kUmmaK * 2), smem_desc_sw128(b_addr + k * kUmmaK * 2),
                              idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_full);
        }
    }
    // What the product is added to is asked for now, under the weight stream (plain epilogue, at most 16 columns a
    // block: the usual case; wider shares load it in store16).
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int a_row = m0 + row_in_tile;
    const bool early_old = kEpi == kPlain && p.swap && cols <= 16;
    // The norm before this product rides on it (tokens are columns here): the scales of the tile's tokens, worked
    // out by the epilogue warps while the weights stream; they meet at the named barrier below before anyone reads.
    __shared__ float s_scale[BN];
    if (warp >= 2 && p.nf.bins_in != nullptr) {
        for (int j = threadIdx.x - 64; j < BN; j += 128) {
            const int tok = n0 + j;
            s_scale[j] = tok < p.rows_b ? 1.0f / sqrtf(bins_total(p.nf.bins_in + (size_t)tok * kBinWords) * (1.0f / (float)p.K) + p.nf.eps)
                                        : 0.0f;
        }
    }
    float old[16];
    if (warp >= 2 && early_old) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int tok = n0 + c_begin + j;
            old[j] = (p.accumulate && j < cols && tok < p.rows_b && a_row < p.rows_a)
                         ? ld_f(p.out, (size_t)tok * p.ldc + a_row, p.out_dt) : 0.0f;
        }
    }
    if (warp >= 2 && p.nf.bins_clear != nullptr && blockIdx.x == 0)   // the norm before: its consumer has run
        for (int i = threadIdx.x - 64; i < p.rows_b * kBinWords; i += 128) p.nf.bins_clear[i] = 0ull;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // all blocks of the cluster are running
    bool received = true;
    if (warp >= 2) {
        // this block's partial tile into its own shared memory, a column at a time (its products are done: the
        // stage ring is free) ...
        const bool ok = kb1 > kb0 ? mbar_wait(acc_full, 0) : true;
        if (!ok && lane == 0) atomicExch(p.status, kTimeoutAccumFull);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            if (ok && kb1 > kb0) {
                tmem_ld32(taddr + (uint32_t)c0, v);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) send[(c0 + j) * kBlockM + row_in_tile] = __uint_as_float(v[j]);
        }
        // ... visible to the copy engine, and when all four warps are there, one thread sends every owner its columns
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
            for (int d = 0; d < S; ++d) {
                const int d_begin = d * BN / S, d_cols = (d + 1) * BN / S - d_begin;
                bulk_copy_to_rank(smem_u32(recv + (size_t)rank * d_cols * kBlockM), smem_u32(send + (size_t)d_begin * kBlockM),
                                  (uint32_t)(d_cols * kBlockM * 4), smem_u32(arrived), (uint32_t)d);
            }
        }
        received = mbar_wait(arrived, 0);
        if (!received && lane == 0) atomicExch(p.status, kTimeoutAccumEmpty);
    }
    // This block has all it was sent; when every block of the cluster says so, no copy is still reading anybody's
    // memory.  The wait comes at the very end.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");   // a meeting in time only: no data rides on it
    if (warp >= 2 && received) {
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
            const int n = min(16, cols - c0);
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            for (int r = 0; r < S; ++r) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j < n) v[j] += recv[(r * cols + c0 + j) * kBlockM + row_in_tile];
            }
            if (p.nf.bins_in != nullptr) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (j < n) v[j] *= s_scale[c_begin + c0 + j];
            }
            if (early_old) {
                // C[token, a_row] = (product + bias) + what was there, as store16 does for this layout
                const bool a_ok = a_row < p.rows_a;
                const float b = p.bias ? ld_f(p.bias, min(a_row, p.rows_a - 1), p.bias_dt) : 0.0f;
                const float g = p.nf.xg_out != nullptr ? ld_f(p.nf.gamma, min(a_row, p.rows_a - 1), p.nf.gamma_dt) : 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = n0 + c_begin + j;
                    const bool ok = j < n && tok < p.rows_b;        // the same for the whole warp
                    const float y = (v[j] + b) + old[j];
                    if (ok && a_ok) st_f(p.out, (size_t)tok * p.ldc + a_row, p.out_dt, y);
                    if (p.nf.xg_out != nullptr && ok) {
                        // the norm after this product rides on it: out * gamma for its consumer, and the token's sum
                        // of squares over this warp's 32 features into the token's exact accumulator
                        if (a_ok) p.nf.xg_out[(size_t)tok * p.rows_a + a_row] = __float2bfloat16(y * g);
                        const float sq = warp_sum(a_ok ? y * y : 0.0f);
                        if (lane == 0) bins_add(p.nf.bins_out + (size_t)tok * kBinWords, sq);
                    }
                }
            } else {
                store16<kEpi>(p, a_row, n0 + c_begin + c0, v, n);
            }
        }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Many tokens: two SMs share one 256 x 256 output tile (tcgen05 cta_group::2).
// With one SM per 128 x 256 tile, every k-block costs 48 KiB of operand traffic
// from L2 into the SM for 512 tensor-core cycles, and the SM's input path, not
// the tensor core, sets the pace.  A pair of SMs multiplies 256 rows of A by
// 256 rows of B: each SM loads its own 128 rows of A but only half of the B
// tile (the tensor cores read the other half from the partner's shared memory),
// 32 KiB per k-block.  The first block of the pair issues the instructions for
// both; operand arrival, stage release and accumulator hand-over are signalled
// across the pair through mbarriers.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// A tile load whose completion is counted by a barrier that may live in the partner block.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
        "[%2];" ::"r"(smem_u32(dst)),
        "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on the barrier at this shared-memory offset in both blocks of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(mask)
        : "memory");
}

// The q/k/v epilogue of one thread: its token's 256 accumulator columns are two whole heads, of which this thread's
// warp takes head `hh`.  Query and key
// heads get the per-head RMS norm (32-bit sum over the head) and the rotation of the pairs (i, i + 64); value
// heads are only rounded.  Queries go to q_out, keys and values to the token's place in the cache pages.
// The same arithmetic as the separate kernel (x * scale * gamma, then the rotation), so prefill and decode
// agree to rounding (crates/nncpu/src/model/forward.rs:278-324).  `row_scale` multiplies the accumulators first: the
// scale of the norm before the projection when that norm rides on this product, else 1 (which changes no bit).
__device__ __forceinline__ void store_qkv_tile(const GemmParams& p, const float (*s_gamma)[128], uint32_t taddr,
                                               int a_row, int n0, float row_scale, int hh) {
    const QkvParams& e = p.qkv;
    const bool row_ok = a_row < p.rows_a;
    // where this token's keys and values go
    long kv_row = -1;
    if (row_ok) {
        const int seq = e.tok_seq[a_row];
        if (seq >= 0) {
            const int pos = e.tok_pos[a_row];
            const int page = e.block_table[(size_t)seq * e.bt_stride + pos / kPage];
            if (page >= 0) kv_row = (long)page * e.n_kv * kPage + pos % kPage;
        }
    }
    {
        const int head = n0 / 128 + hh;
        if (head >= e.n_heads + 2 * e.n_kv) return;
        const bool is_q = head < e.n_heads, is_k = !is_q && head < e.n_heads + e.n_kv;
        const uint32_t t0 = taddr + (uint32_t)(128 * hh);
        const void* gamma = is_q ? e.q_gamma : (is_k ? e.k_gamma : nullptr);
        float scale = 1.0f;
        if (gamma) {
            float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 64) {
                uint32_t u[64];
                tmem_ld64(t0 + (uint32_t)c0, u);
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const float x = __uint_as_float(u[c]) * row_scale;
                    ss[c & 3] = fmaf(x, x, ss[c & 3]);
                }
            }
            scale = 1.0f / sqrtf(((ss[0] + ss[1]) + (ss[2] + ss[3])) * (1.0f / 128.0f) + e.eps);
        }
        __nv_bfloat16* dst = nullptr;
        if (row_ok) {
            if (is_q) {
                dst = e.q_out + ((size_t)a_row * e.n_heads + head) * 128;
            } else if (kv_row >= 0) {
                const int kvh = is_k ? head - e.n_heads : head - e.n_heads - e.n_kv;
                dst = (is_k ? e.k_pages : e.v_pages) + ((size_t)kv_row + (size_t)kvh * kPage) * 128;
            }
        }
        const bool rotate = (is_q || is_k) && e.cos_sin != nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t lo[32], hi[32];   // dimensions c0 .. c0 + 31 and their partners 64 on
            tmem_ld32(t0 + (uint32_t)c0, lo);
            tmem_ld32(t0 + (uint32_t)(64 + c0), hi);
            if (dst == nullptr) continue;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                float a = __uint_as_float(lo[c]) * row_scale, b = __uint_as_float(hi[c]) * row_scale;
                if (gamma) {
                    a = (a * scale) * s_gamma[is_q ? 0 : 1][c0 + c];
                    b = (b * scale) * s_gamma[is_q ? 0 : 1][64 + c0 + c];
                }
                if (rotate) {
                    const float2 cs = e.cos_sin[(size_t)(c0 + c) * p.rows_a + a_row];   // lanes are tokens
                    const float ra = cs.x * a - cs.y * b, rb = cs.y * a + cs.x * b;
                    a = ra;
                    b = rb;
                }
                lo[c] = __float_as_uint(a);
                hi[c] = __float_as_uint(b);
            }
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
                uint4 w;
                __nv_bfloat162 h2;
                h2 = __floats2bfloat162_rn(__uint_as_float(lo[c]), __uint_as_float(lo[c + 1])); w.x = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(lo[c + 2]), __uint_as_float(lo[c + 3])); w.y = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(lo[c + 4]), __uint_as_float(lo[c + 5])); w.z = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(lo[c + 6]), __uint_as_float(lo[c + 7])); w.w = *reinterpret_cast<uint32_t*>(&h2);
                *reinterpret_cast<uint4*>(dst + c0 + c) = w;
                h2 = __floats2bfloat162_rn(__uint_as_float(hi[c]), __uint_as_float(hi[c + 1])); w.x = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(hi[c + 2]), __uint_as_float(hi[c + 3])); w.y = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(hi[c + 4]), __uint_as_float(hi[c + 5])); w.z = *reinterpret_cast<uint32_t*>(&h2);
                h2 = __floats2bfloat162_rn(__uint_as_float(hi[c + 6]), __uint_as_float(hi[c + 7])); w.w = *reinterpret_cast<uint32_t*>(&h2);
                *reinterpret_cast<uint4*>(dst + 64 + c0 + c) = w;
            }
        }
    }
}

template <int kStages, int kEpi>
__global__ void __launch_bounds__(kPairThreads)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
    constexpr int BN = 256;                       // columns of the pair's tile; each block stages 128 of its B rows
    constexpr int kBytesA = kBlockM * kBlockK * 2;
    constexpr int kBytesB = (BN / 2) * kBlockK * 2;
    constexpr int kTmemCols = 2 * BN;             // two accumulators of 128 lanes x 256 columns per block
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kBytesA;
    uint64_t* full = (uint64_t*)(smem_b + kStages * kBytesB);   // used in the first block: both blocks' loads
    uint64_t* empty = full + kStages;                           // in each block: its stage may be refilled
    uint64_t* acc_full = empty + kStages;                       // [2] in each block
    uint64_t* acc_empty = acc_full + 2;                         // [2] used in the first block: both epilogues
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    __shared__ float s_gamma[kEpi == kQkv ? 2 : 1][128];   // the q and k norm weights of the fused q/k/v epilogue
    let_next_kernel_start();   // the set-up below runs while the kernel before this one ends
    if constexpr (kEpi == kQkv) {
        for (int i = threadIdx.x; i < 256; i += kPairThreads) {
            const void* gamma = i < 128 ? p.qkv.q_gamma : p.qkv.k_gamma;
            s_gamma[i >> 7][i & 127] = gamma ? ld_f(gamma, i & 127, p.qkv.g_dt) : 1.0f;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_items = p.tiles_a * p.tiles_b;    // tiles of 256 x 256

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);       // the first block's loader arrives and announces both blocks' bytes
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 16); // eight epilogue warps in each block
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    cluster_barrier();   // both blocks' barriers exist before anyone signals across the pair
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    wait_for_previous_kernels();

    if (warp == 0) {
        if (lane == 0) {
            int kb_run = 0;
            bool ok = true;
            for (int w = pair; w < n_items && ok; w += n_pairs) {
                const int m0 = (w % p.tiles_a) * 256 + (int)rank * kBlockM;
                const int n0 = (w / p.tiles_a) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < p.kb_total; ++kb, ++kb_run) {
                    const int s = kb_run % kStages;
                    if (!mbar_wait(&empty[s], ((kb_run / kStages) & 1) ^ 1)) {
                        atomicExch(p.status, kTimeoutEmpty);
                        ok = false;
                        break;
                    }
                    // The partner's copies are counted by the first block's barrier too.  They cannot complete a
                    // phase early: the phase also needs the first block's own arrival, and a stage is refilled
                    // only after the instructions that read it have retired in both blocks.
                    const uint32_t bar = map_to_rank(smem_u32(&full[s]), 0);
                    if (leader) mbar_expect_tx(&full[s], 2 * (kBytesA + kBytesB));
                    tma_load_2d_pair(smem_a + s * kBytesA, &map_a, bar, kb * kBlockK, m0);
                    tma_load_2d_pair(smem_b + s * kBytesB, &map_b, bar, kb * kBlockK, n0);
                }
            }
            if (!ok) {
                // copies already in flight are counted by the first block's barriers; give them time to land
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc_bf16(256, BN);
            int kb_run = 0, it = 0;
            bool ok = true;
            for (int w = pair; w < n_items && ok; w += n_pairs, ++it) {
                const int buf = it & 1;
                if (!mbar_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, kTimeoutAccumEmpty);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < p.kb_total; ++kb, ++kb_run) {
                    const int s = kb_run % kStages;
                    if (!mbar_wait(&full[s], (kb_run / kStages) & 1)) {
                        atomicExch(p.status, kTimeoutFull);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem_a + s * kBytesA);
                    const uint32_t b_addr = smem_u32(smem_b + s * kBytesB);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k)
                        umma_bf16_pair(tmem_d, smem_desc_sw128(a_addr + k * kUmmaK * 2),
                                       smem_desc_sw128(b_addr + k * kUmmaK * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;         // the quarter of the tensor-memory lanes this warp may read
        const int half = (warp - 2) >> 2;     // the half of the tile's columns it takes
        const int row_in_tile = quarter * 32 + lane;
        int it = 0;
        for (int w = pair; w < n_items; w += n_pairs, ++it) {
            const int m0 = (w % p.tiles_a) * 256 + (int)rank * kBlockM;
            const int n0 = (w / p.tiles_a) * BN;
            const int a_row = m0 + row_in_tile;
            const int buf = it & 1;
            if (!mbar_wait(&acc_full[buf], (it >> 1) & 1)) {
                if (lane == 0) atomicExch(p.status, kTimeoutAccumFull);
                break;
            }
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN);
            // the norm before this product rides on it: its rows' scales multiply the accumulators
            const bool a_ok = a_row < p.rows_a;
            float row_scale = 1.0f;
            if (p.nf.bins_in != nullptr && a_ok)
                row_scale = 1.0f / sqrtf(bins_total(p.nf.bins_in + (size_t)a_row * kBinWords) * (1.0f / (float)p.K) + p.nf.eps);
            if constexpr (kEpi == kQkv) {
                store_qkv_tile(p, s_gamma, taddr, a_row, n0, row_scale, half);
            } else if (kEpi == kPlain && p.nf.xg_out != nullptr) {
                // the norm after this product rides on it: besides out (float32, rows of whole 16-byte pieces: the
                // launcher checked) it leaves out * gamma in bfloat16 and adds this tile's part of the row's sum of
                // squares to the row's accumulator
                float ss = 0.0f;
#pragma unroll 1
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 16) {
                    const int col = n0 + c0;
                    if (col >= p.rows_b) break;        // the same for the whole warp
                    float v[16];
                    tmem_ld16(taddr + (uint32_t)c0, v);   // every lane takes part in the load, whatever its row
                    if (!a_ok) continue;
                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)a_row * p.ldc + col);
                    float4 y[4];
                    if (p.accumulate) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) y[j] = dst[j];
                    }
                    float g[16];
                    if (p.nf.gamma_dt == DT_BF16) {
                        const uint4* gp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.nf.gamma) + col);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint4 w = gp[h];
                            const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __bfloat1622float2(wh[j]);
                                g[8 * h + 2 * j] = f.x;
                                g[8 * h + 2 * j + 1] = f.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) g[j] = reinterpret_cast<const float*>(p.nf.gamma)[col + j];
                    }
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += ld_f(p.bias, col + j, p.bias_dt);
                    }
                    if (p.accumulate) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            v[4 * j] += y[j].x; v[4 * j + 1] += y[j].y; v[4 * j + 2] += y[j].z; v[4 * j + 3] += y[j].w;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    __nv_bfloat16* xg = p.nf.xg_out + (size_t)a_row * p.rows_b + col;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        __nv_bfloat162 o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            o[j] = __floats2bfloat162_rn(v[8 * h + 2 * j] * g[8 * h + 2 * j], v[8 * h + 2 * j + 1] * g[8 * h + 2 * j + 1]);
                        *reinterpret_cast<uint4*>(xg + 8 * h) = *reinterpret_cast<uint4*>(o);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) ss = fmaf(v[j], v[j], ss);
                }
                if (a_ok) {
                    bins_add(p.nf.bins_out + (size_t)a_row * kBinWords, ss);
                    if (p.nf.bins_clear != nullptr && n0 == 0 && half == 0) {
                        // the accumulators of the norm before, whose consumer has run: zero for their next use
                        uint4* z = reinterpret_cast<uint4*>(p.nf.bins_clear + (size_t)a_row * kBinWords);
#pragma unroll
                        for (int j = 0; j < kBinWords / 2; ++j) z[j] = make_uint4(0, 0, 0, 0);
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= row_scale;
                    store16<kEpi>(p, a_row, n0 + c0, v);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[buf]), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    cluster_barrier();   // the partner may still be reading this block's half of B, or signalling its barriers
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps (cached by what they describe) and the launcher.
// ---------------------------------------------------------------------------

// A [rows, K] bfloat16 matrix with row stride `ld` elements, cut in boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* base, int rows, int K, long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    NN_CHECK(fn != nullptr, "gemm: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NN_CHECK(r == CUDA_SUCCESS, "gemm: cuTensorMapEncodeTiled failed with code %d (rows %d, K %d, ld %ld, box %d)",
             (int)r, rows, K, ld, box_rows);
    return 0;
}

struct MapCache {
    std::mutex lock;
    std::map<std::tuple<const void*, int, int, long, int>, CUtensorMap> maps;

    int get(CUtensorMap* out, const void* base, int rows, int K, long ld, int box_rows) {
        std::lock_guard<std::mutex> g(lock);
        const auto key = std::make_tuple(base, rows, K, ld, box_rows);
        auto it = maps.find(key);
        if (it == maps.end()) {
            CUtensorMap m;
            if (int e = make_map(&m, base, rows, K, ld, box_rows)) return e;
            if (maps.size() > 65536) maps.clear();
            it = maps.emplace(key, m).first;
        }
        *out = it->second;
        return 0;
    }
};

MapCache g_maps;

int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

template <int BN, int kStages>
constexpr size_t smem_bytes() {
    return 1024 + (size_t)kStages * (kBlockM * kBlockK * 2 + BN * kBlockK * 2) + (2 * kStages + 4) * sizeof(uint64_t) + 16;
}

template <int BN, int kStages, int kEpi>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int blocks_per_sm, cudaStream_t stream) {
    constexpr size_t smem = smem_bytes<BN, kStages>();
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, kStages, kEpi>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        NN_CHECK(e == cudaSuccess, "gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    const int n_items = p.tiles_a * p.tiles_b;
    const int grid = n_items < blocks_per_sm * sm_count() ? n_items : blocks_per_sm * sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = overlap_attribute(attr);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, kStages, kEpi>, ma, mb, p);
    NN_CHECK(e == cudaSuccess, "gemm: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

template <int BN, int kStages, int kEpi, int kTM = 1>
int launch_streamk(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    constexpr size_t smem = smem_bytes<BN, kStages>() + (size_t)kStages * (kTM - 1) * (kBlockM * kBlockK * 2);
    static_assert(smem <= 227 * 1024, "the stages fit shared memory");
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_streamk_kernel<BN, kStages, kEpi, kTM>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        NN_CHECK(e == cudaSuccess, "gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    // one block per SM with a deep pipeline; at least 4 k-blocks per block
    const long units = (long)p.tiles_a * p.tiles_b * p.kb_total;
    long grid = sm_count();
    if (grid > units / 4) grid = units / 4;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = overlap_attribute(attr);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_streamk_kernel<BN, kStages, kEpi, kTM>, ma, mb, p);
    NN_CHECK(e == cudaSuccess, "gemm (stream-K): launch failed: %s", cudaGetErrorString(e));
    if (units % grid != 0 || (units / grid) % p.kb_total != 0) {
        // some tile is shared between blocks
        cudaLaunchConfig_t fix = {};
        fix.gridDim = dim3((unsigned)(p.tiles_a * p.tiles_b), BN / 16, kTM);
        fix.blockDim = dim3(kBlockM);
        fix.stream = stream;
        cudaLaunchAttribute fix_attr[1];
        fix.attrs = fix_attr;
        fix.numAttrs = overlap_attribute(fix_attr);
        const cudaError_t e2 = cudaLaunchKernelEx(&fix, gemm_streamk_fixup_kernel<BN, kEpi, kTM>, p, (int)grid);
        NN_CHECK(e2 == cudaSuccess, "gemm (stream-K, adding the parts): launch failed: %s", cudaGetErrorString(e2));
    }
    return 0;
}

template <int kEpi>
int dispatch_streamk(int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    switch (bn) {
        case 16: return launch_streamk<16, 10, kEpi>(ma, mb, p, stream);
        case 32: return launch_streamk<32, 10, kEpi>(ma, mb, p, stream);
        case 64: return launch_streamk<64, 8, kEpi>(ma, mb, p, stream);
        case 128: return launch_streamk<128, 6, kEpi>(ma, mb, p, stream);
        default: return launch_streamk<256, 4, kEpi>(ma, mb, p, stream);
    }
}

// The same with 256 rows of A per unit (p.tiles_a counts those).
template <int kEpi>
int dispatch_streamk_wide(int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    if (bn == 128) return launch_streamk<128, 4, kEpi, 2>(ma, mb, p, stream);
    return launch_streamk<256, 3, kEpi, 2>(ma, mb, p, stream);
}

template <int BN, int kStages, int kEpi>
int launch_cluster(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    constexpr size_t smem = cluster_smem_bytes<BN, kStages>();
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_cluster_kernel<BN, kStages, kEpi>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        NN_CHECK(e == cudaSuccess, "gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.tiles_a * p.tiles_b * p.splits));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1 + overlap_attribute(attr + 1);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_cluster_kernel<BN, kStages, kEpi>, ma, mb, p);
    NN_CHECK(e == cudaSuccess, "gemm (cluster of %d): launch failed: %s", p.splits, cudaGetErrorString(e));
    return 0;
}

template <int kStages, int kEpi>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)kStages * (kBlockM * kBlockK * 2 + 128 * kBlockK * 2) +
                            (2 * kStages + 4) * sizeof(uint64_t) + 16;
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<kStages, kEpi>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        NN_CHECK(e == cudaSuccess, "gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    const int n_items = p.tiles_a * p.tiles_b;
    const int max_pairs = sm_count() / 2;
    const int pairs = n_items < max_pairs ? n_items : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1 + overlap_attribute(attr + 1);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<kStages, kEpi>, ma, mb, p);
    NN_CHECK(e == cudaSuccess, "gemm (pairs of SMs): launch failed: %s", cudaGetErrorString(e));
    return 0;
}

template <int kEpi>
int dispatch_cluster(int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    switch (bn) {
        // stages chosen so that two blocks share an SM up to 64 tokens (ring + receive buffer below 110 KB)
        case 32: return launch_cluster<32, 4, kEpi>(ma, mb, p, stream);
        case 64: return launch_cluster<64, 3, kEpi>(ma, mb, p, stream);
        default: return launch_cluster<128, 3, kEpi>(ma, mb, p, stream);
    }
}

template <int kEpi>
int dispatch(int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, cudaStream_t stream) {
    switch (bn) {
        case 16: return launch<16, 4, kEpi>(ma, mb, p, 3, stream);
        case 32: return launch<32, 4, kEpi>(ma, mb, p, 2, stream);
        case 64: return launch<64, 4, kEpi>(ma, mb, p, 2, stream);
        case 128: return launch<128, 6, kEpi>(ma, mb, p, 1, stream);
        default: return launch<256, 4, kEpi>(ma, mb, p, 1, stream);
    }
}

}  // namespace

// Whether nncpu_linear_tc takes these sizes: both row strides must keep TMA's
// 16-byte rule, which for bfloat16 means multiples of 8 elements.
extern "C" int nncpu_linear_tc_supported(int M, int N, int K, int lda) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0;
}

// Floats of scratch a workspace must hold for any product this library launches.
extern "C" long nncpu_linear_tc_scratch_floats() { return 20l << 20; }  // 80 MiB: two partial units of 2 x 256 x 128 per SM

// The q/k/v projection of a prompt with its epilogue fused: X[M, K] . W[(n_heads + 2 n_kv) * 128, K]^T, then per
// head the RMS norm (q and k, if their weights are given), the rotation (if cos_sin is given) and the stores:
// queries to q_out [M, n_heads * 128], keys and values to each token's row of the cache pages.  No bias.
extern "C" int nncpu_linear_tc_qkv_supported(int M, int K, int lda, int n_heads, int n_kv, int head_dim) {
    return M >= 512 && K > 0 && K % 8 == 0 && lda % 8 == 0 && head_dim == 128 && n_heads > 0 && n_kv > 0 &&
           n_heads % 2 == 0 && n_kv % 2 == 0;
}

extern "C" int nncpu_linear_tc_qkv(const void* X, const void* W, int M, int K, int lda, void* q_out, void* k_pages,
                                   void* v_pages, const void* q_gamma, const void* k_gamma, int g_dt, float eps,
                                   const float* cos_sin, const int* tok_seq, const int* tok_pos, const int* block_table,
                                   int bt_stride, int n_heads, int n_kv, int head_dim, const void* bins_in,
                                   float norm_eps, int* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(nncpu_linear_tc_qkv_supported(M, K, lda, n_heads, n_kv, head_dim),
             "gemm (q/k/v epilogue): M %d, K %d, lda %d, %d heads over %d of size %d: it takes 512 or more tokens, "
             "head size 128, even head counts, K and lda multiples of 8", M, K, lda, n_heads, n_kv, head_dim);
    NN_CHECK(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)q_out % 16) == 0 &&
             ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0,
             "gemm (q/k/v epilogue): operands must be 16-byte aligned");
    NN_CHECK(tok_seq && tok_pos && block_table && status, "gemm (q/k/v epilogue): token places and status are needed");
    NN_CHECK((uintptr_t)cos_sin % 8 == 0, "gemm (q/k/v epilogue): the rotation table must be 8-byte aligned (cos/sin pairs)");
    const int N = (n_heads + 2 * n_kv) * 128;
    GemmParams p{};
    p.K = K;
    p.kb_total = (K + kBlockK - 1) / kBlockK;
    p.status = status;
    p.swap = 0;
    p.rows_a = M; p.rows_b = N;
    p.tiles_a = (M + 255) / 256;
    p.tiles_b = N / 256;
    p.splits = 1;
    p.qkv.q_out = (__nv_bfloat16*)q_out;
    p.qkv.k_pages = (__nv_bfloat16*)k_pages;
    p.qkv.v_pages = (__nv_bfloat16*)v_pages;
    p.qkv.q_gamma = q_gamma; p.qkv.k_gamma = k_gamma; p.qkv.g_dt = g_dt; p.qkv.eps = eps;
    p.qkv.cos_sin = (const float2*)cos_sin;
    p.qkv.tok_seq = tok_seq; p.qkv.tok_pos = tok_pos; p.qkv.block_table = block_table; p.qkv.bt_stride = bt_stride;
    p.qkv.n_heads = n_heads; p.qkv.n_kv = n_kv;
    if (bins_in != nullptr) {
        // X holds a norm's rows times gamma; the rows' scales multiply the accumulators (see nncpu_linear_tc)
        NN_CHECK(((uintptr_t)bins_in % 8) == 0 && norm_eps >= 0.0f, "gemm (q/k/v epilogue): a norm's accumulators (8-byte aligned), eps %g",
                 norm_eps);
        p.nf.bins_in = (const unsigned long long*)bins_in;
        p.nf.eps = norm_eps;
    }
    CUtensorMap ma, mb;
    if (int e = g_maps.get(&ma, X, M, K, lda, kBlockM)) return e;
    if (int e = g_maps.get(&mb, W, N, K, K, 128)) return e;
    return launch_pair<6, kQkv>(ma, mb, p, stream);
}

// The library's check of its own failure path: one 128 x 256 tile of X[128, K] . W[256, K]^T through the persistent
// kernel, whose stage barriers are told to expect 16 bytes more than the copies bring and whose waits are limited to
// `limit_ms` instead of two seconds.  Every role of the block runs into its limit, the copies in flight are waited
// for, tensor memory is freed, and the kernel returns with *status set: nothing traps, faults or waits without
// bound, and the workspace serves the next product as before.  `out` (float [128, 256]) is not written.
extern "C" int nncpu_linear_tc_wait_probe(const void* X, const void* W, float* out, int K, int limit_ms, int* status,
                                          void* stream_) {
    NN_CHECK(K >= 64 && K % 64 == 0 && K <= 4096, "gemm wait probe: K %d (a multiple of 64 up to 4096)", K);
    NN_CHECK(limit_ms >= 1 && limit_ms <= 1000, "gemm wait probe: a limit of %d ms (1 to 1000)", limit_ms);
    NN_CHECK(X && W && out && status, "gemm wait probe: operands and the status word are needed");
    NN_CHECK(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm wait probe: operands must be 16-byte aligned");
    GemmParams p{};
    p.K = K;
    p.kb_total = K / kBlockK;
    p.out = out; p.out_dt = DT_F32; p.ldc = 256; p.status = status;
    p.rows_a = 128; p.rows_b = 256; p.tiles_a = 1; p.tiles_b = 1; p.splits = 1;
    p.wait_ns = (unsigned long long)limit_ms * 1000000ull;
    p.tx_extra = 16;
    CUtensorMap ma, mb;
    if (int e = g_maps.get(&ma, X, 128, K, K, kBlockM)) return e;
    if (int e = g_maps.get(&mb, W, 256, K, K, 256)) return e;
    return launch<256, 4, kPlain>(ma, mb, p, 1, (cudaStream_t)stream_);
}

// C[M, N] (+)= X[M, K] . W[N, K]^T + bias, or with epilogue 1: C[M, N/2] = silu(gate) * up for W rows
// interleaved in blocks of 8 (8 gate rows, the 8 up rows of the same outputs, ...).  X and W are
// bfloat16; C is float or bfloat16 with row stride ldc.  `scratch` (nncpu_linear_tc_scratch_floats
// floats) serves the products that deal their k-blocks out evenly; launches that share it must not
// overlap on the GPU.  `status` is a device word that a kernel sets when one of its bounded waits ran out.
// `plan` chooses among the kernels where a measurement or a test wants another one than the sizes would get:
// 0 the default (products of 512 or more tokens on pairs of SMs with 256 x 256 tiles; 65 to 256 tokens with their
// k-blocks dealt out evenly over the SMs; 17 to 64 tokens a cluster per output tile); kPlanEvenFrom17: dealt out
// evenly from 17 tokens on; kPlanNeverEven: never dealt out evenly; kPlanNoPairs: one SM per 128 x 256 tile;
// kPlanNarrowUnits: units of 128 weight rows where 256 would be taken.
enum Plan : int { kPlanEvenFrom17 = 1, kPlanNeverEven = 2, kPlanNoPairs = 4, kPlanNarrowUnits = 8 };

//
// The norms around a product of whole prompts can ride on it as they do on the few-token products (linear_skinny.cu),
// where nncpu_linear_tc_fuses_norms(M, N) says so (the kernel for pairs of SMs).  Producer (plain epilogue, float32
// C with 16-byte rows, N a multiple of 16): xg_out bfloat16 [M, N] receives C * gamma and bins_out [M, 16] (64-bit
// words, zero before the call) the exact sums of squares of C's rows; bins_clear [M, 16] (or null) is set to zero.
// Consumer: X holds such rows of width K and bins_in [M, 16] their accumulators: the result is multiplied by
// 1 / sqrt(sum / K + eps) per row before bias and activation.
// From 17 to 64 tokens the same holds where nncpu_linear_tc_norm_roles says so (bit 0: may be a consumer, bit 1: may
// be a producer): the cluster kernel does both (a producer with at most 16 tokens a block), the kernel of whole
// 128-row tiles per block consumes.
extern "C" int nncpu_linear_tc_fuses_norms(int M, int N) { return M >= 512 && N >= 512; }

namespace {
// The cluster size that nncpu_linear_tc picks for a product of 17 to 64 tokens (1: whole tiles per block).
int cluster_blocks(int bn, int n_tiles, int kb_total) {
    if (!(bn >= 32 && bn <= 128 && n_tiles < sm_count())) return 1;
    const int places = (bn <= 64 ? 2 : 1) * sm_count() * 87 / 100;
    int best = 1;
    for (int s = 2; s <= 8 && s <= bn && kb_total / s >= 4; ++s)
        if (n_tiles * s <= places) best = s;
    return best;
}
}  // namespace

extern "C" int nncpu_linear_tc_norm_roles(int M, int N, int K) {
    if (nncpu_linear_tc_fuses_norms(M, N)) return 3;
    if (M < 17 || M > 64) return 0;
    const int bn = M <= 32 ? 32 : 64;
    const int s = cluster_blocks(bn, (N + kBlockM - 1) / kBlockM, (K + kBlockK - 1) / kBlockK);
    return 1 | ((s > 1 && (bn + s - 1) / s <= 16) ? 2 : 0);
}

extern "C" int nncpu_linear_tc(const void* X, const void* W, const void* bias, int bias_dt, void* C, int c_dt, int M,
                               int N, int K, int lda, int ldc, int accumulate, int epilogue, int plan, void* xg_out,
                               const void* gamma, int gamma_dt, void* bins_out, void* bins_clear, const void* bins_in,
                               float eps, float* scratch, int* status, void* stream_) {
    const int streamk_mode = (plan & kPlanNeverEven) ? 0 : (plan & kPlanEvenFrom17) ? 2 : 1;
    const int pair_mode = (plan & kPlanNoPairs) ? 0 : 1;
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(nncpu_linear_tc_supported(M, N, K, lda),
             "gemm: M %d, N %d, K %d, lda %d: K and lda must be multiples of 8 for the tensor-core path", M, N, K, lda);
    NN_CHECK(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm: operands must be 16-byte aligned");
    NN_CHECK(epilogue == kPlain || epilogue == kSwiglu, "gemm: unknown epilogue %d", epilogue);
    const int n_out = epilogue == kSwiglu ? N / 2 : N;
    NN_CHECK(ldc >= n_out, "gemm: ldc %d is below the %d output features", ldc, n_out);
    if (epilogue == kSwiglu)
        NN_CHECK(N % 16 == 0 && bias == nullptr && !accumulate,
                 "gemm: the gated epilogue needs N %% 16 == 0, no bias and no accumulation (N %d)", N);
    GemmParams p{};
    p.K = K;
    p.kb_total = (K + kBlockK - 1) / kBlockK;
    p.out = C; p.bias = bias; p.out_dt = c_dt; p.bias_dt = bias_dt; p.ldc = ldc; p.accumulate = accumulate;
    p.scratch = scratch; p.status = status;
    const int esize = c_dt == DT_F32 ? 4 : 2;
    p.vec = ((uintptr_t)C % 16 == 0) && ((size_t)ldc * esize % 16 == 0);
    if (xg_out != nullptr || bins_in != nullptr) {
        const int roles = plan == 0 ? nncpu_linear_tc_norm_roles(M, N, K) : (nncpu_linear_tc_fuses_norms(M, N) && !(plan & kPlanNoPairs) ? 3 : 0);
        NN_CHECK((bins_in == nullptr || (roles & 1)) && (xg_out == nullptr || (roles & 2)),
                 "gemm: this product cannot carry that norm (M %d, N %d, K %d: see nncpu_linear_tc_norm_roles)", M, N, K);
        NN_CHECK(xg_out == nullptr || bins_in == nullptr, "gemm: a product is a norm's producer or its consumer");
    }
    if (xg_out != nullptr) {
        NN_CHECK(epilogue == kPlain && c_dt == DT_F32 && (p.vec || M <= 64) && N % 16 == 0 && gamma != nullptr && bins_out != nullptr &&
                     ((uintptr_t)xg_out % 16) == 0 && ((uintptr_t)gamma % 16) == 0 && ((uintptr_t)bins_out % 16) == 0 &&
                     ((uintptr_t)bins_clear % 16) == 0,
                 "gemm: leaving a norm's input needs the plain epilogue, float32 output in 16-byte rows, N %% 16 == 0, "
                 "the norm's weights and its accumulators (all 16-byte aligned)");
        p.nf.xg_out = (__nv_bfloat16*)xg_out;
        p.nf.gamma = gamma;
        p.nf.gamma_dt = gamma_dt;
        p.nf.bins_out = (unsigned long long*)bins_out;
        p.nf.bins_clear = (unsigned long long*)bins_clear;
    }
    if (bins_in != nullptr) {
        NN_CHECK(((uintptr_t)bins_in % 8) == 0 && eps >= 0.0f, "gemm: a norm's accumulators (8-byte aligned), eps %g", eps);
        p.nf.bins_in = (const unsigned long long*)bins_in;
        p.nf.eps = eps;
    }
    CUtensorMap ma, mb;
    int bn;
    if (M <= 256) {
        // few tokens: weights are the 128-row operand, tokens the narrow one
        p.swap = 1;
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        p.rows_a = N; p.rows_b = M;
        if (int e = g_maps.get(&ma, W, N, K, K, kBlockM)) return e;
        if (int e = g_maps.get(&mb, X, M, K, lda, bn)) return e;
    } else {
        p.swap = 0;
        bn = N >= 256 ? 256 : 128;
        p.rows_a = M; p.rows_b = N;
        if (int e = g_maps.get(&ma, X, M, K, lda, kBlockM)) return e;
        if (M >= 512 && N >= 512 && pair_mode) {
            // enough work for 256 x 256 tiles on pairs of SMs
            if (int e = g_maps.get(&mb, W, N, K, K, 128)) return e;
            p.tiles_a = (M + 255) / 256;
            p.tiles_b = (N + 255) / 256;
            p.splits = 1;
            return epilogue == kSwiglu ? launch_pair<6, kSwiglu>(ma, mb, p, stream)
                                       : launch_pair<6, kPlain>(ma, mb, p, stream);
        }
        if (int e = g_maps.get(&mb, W, N, K, K, bn)) return e;
    }
    p.tiles_a = (p.rows_a + kBlockM - 1) / kBlockM;
    p.tiles_b = (p.rows_b + bn - 1) / bn;
    const int n_tiles = p.tiles_a * p.tiles_b;
    p.splits = 1;
    // Up to 16 tokens (the few-token kernel of linear_skinny.cu is the product path for those; this serves direct
    // calls) and 65 to 256 tokens: the work is cut evenly over the SMs; 17 to 64: a cluster per output tile (measured:
    // at 96 tokens 139 us against 220 us for the four products of a Qwen3-8B layer, at 64 tokens 123 against 117)
    // The same for 257 and more tokens that do not fill the SMs with 128 x 256 tiles at least twice.
    const bool even_swap = p.swap && (bn <= 16 || bn >= (streamk_mode == 2 ? 32 : 128));
    const bool even_plain = !p.swap && n_tiles < 2 * sm_count();
    if ((even_swap || even_plain) && streamk_mode && scratch != nullptr &&
        2l * sm_count() * bn * kBlockM <= nncpu_linear_tc_scratch_floats()) {
        p.splits = 1;
        // 65 to 256 tokens: a k-block of the tokens is as large as a tile of the weights or twice that, so units of
        // 256 weight rows, which copy it once for two tiles.  Only with tiles for every SM: below that every unit is
        // left in parts, and parts of twice the size cost more than the copies save (measured at 128 tokens on the
        // Qwen3-8B layer sizes: 24 576 rows 57.6 -> 55.5 us, at 256 tokens 78.0 -> 71.5; 4 096 rows 18.3 -> 23.2 us)
        if (p.swap && bn >= 128 && n_tiles >= sm_count() && !(plan & kPlanNarrowUnits) &&
            4l * sm_count() * bn * kBlockM <= nncpu_linear_tc_scratch_floats()) {
            p.tiles_a = (p.rows_a + 2 * kBlockM - 1) / (2 * kBlockM);
            return epilogue == kSwiglu ? dispatch_streamk_wide<kSwiglu>(bn, ma, mb, p, stream)
                                       : dispatch_streamk_wide<kPlain>(bn, ma, mb, p, stream);
        }
        return epilogue == kSwiglu ? dispatch_streamk<kSwiglu>(bn, ma, mb, p, stream)
                                   : dispatch_streamk<kPlain>(bn, ma, mb, p, stream);
    }
    if (p.swap && bn >= 32 && bn <= 128 && n_tiles < sm_count()) {
        // Few tokens, fewer tiles than SMs: a cluster of S blocks shares an output tile, each block a slice of K.
        // S is the largest cluster (up to 8, at least 4 k-blocks a slice) whose blocks all run at once with room
        // to spare: clusters are placed inside one GPC, and a grid that counts on the last free places leaves
        // whole clusters waiting (measured at 64 tokens on the Qwen3-8B layer sizes: 48 tiles take 5 blocks each,
        // 17.3 us, where 6 take 25 us; 32 tiles take 8).  With as many tiles as SMs or more, whole tiles per block
        // stream as fast and need no exchange.
        const int best = cluster_blocks(bn, n_tiles, p.kb_total);
        p.splits = best;
        if (best > 1)
            return epilogue == kSwiglu ? dispatch_cluster<kSwiglu>(bn, ma, mb, p, stream)
                                       : dispatch_cluster<kPlain>(bn, ma, mb, p, stream);
    }
    return epilogue == kSwiglu ? dispatch<kSwiglu>(bn, ma, mb, p, stream) : dispatch<kPlain>(bn, ma, mb, p, stream);
}
