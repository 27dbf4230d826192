// bfloat16 matrix product for sm_100a on the 5th-generation tensor cores:
//   C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias[N])
// Operand tiles are brought to shared memory by TMA (128-byte swizzle), one
// elected thread issues tcgen05.mma with the accumulator in tensor memory,
// and four warps read the accumulator back with tcgen05.ld for the epilogue.
//
// One kernel serves prefill and decode.  The tensor-core M operand is always a
// 128-row tile of "A" and the N operand a BN-row tile of "B":
//   * many tokens:  A = activations, B = weights           (C tile = A rows x B rows)
//   * few tokens:   A = weights,     B = activations, and the epilogue stores
//     the tile transposed, so every weight byte is read once and no tensor
//     core row is wasted on padding.
// The reference computes the same products with its own BF16 row kernels
// (crates/nncpu/src/kernels/mod.rs:454-485, crates/nncpu/src/kernels/scalar.rs:555-567);
// accumulation is 32-bit here as there.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *status and
// the block leaves through the common exit, which frees its tensor memory.

#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

#define NN_LIB gemm_sm100
#include "common.cuh"

namespace {

constexpr int kBlockM = 128;  // rows of the A tile = tensor-core M
constexpr int kBlockK = 64;   // 64 bfloat16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;    // K of one tcgen05.mma for 16-bit inputs
constexpr uint32_t kSpinLimit = 1u << 26;
constexpr int kThreads = 192;  // warp 0: TMA, warp 1: MMA and tensor memory, warps 2-5: epilogue

enum GemmStatus : int { kOk = 0, kTimeoutEmpty = 101, kTimeoutFull = 102, kTimeoutAccum = 103 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// swizzled in 128-byte mode: groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);  // start address
    d |= (uint64_t)1 << 16;                  // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
    d |= (uint64_t)1 << 46;                  // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                  // 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 inputs, float accumulator, both operands K-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct EpilogueArgs {
    void* out;         // [rows of the token operand, ldc]
    const void* bias;  // per output feature, or null
    int out_dt, bias_dt;
    int ldc;
    int accumulate;  // add to what `out` holds
    int swap;        // 0: A rows are tokens; 1: A rows are output features
};

template <int BN, int kStages>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, int rows_a,
                 int rows_b, int K, EpilogueArgs ep, int* __restrict__ status) {
    constexpr int kBytesA = kBlockM * kBlockK * 2;
    constexpr int kBytesB = BN * kBlockK * 2;
    constexpr int kTmemCols = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + kStages * kBytesA;
    uint64_t* full = (uint64_t*)(smem_b + kStages * kBytesB);
    uint64_t* empty = full + kStages;
    uint64_t* accum_full = empty + kStages;
    uint32_t* tmem_slot = (uint32_t*)(accum_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kBlockM, n0 = blockIdx.y * BN;
    const int num_kb = (K + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum_full, 1);
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

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % kStages;
                const uint32_t phase = (kb / kStages) & 1;
                if (!mbar_wait(&empty[s], phase ^ 1)) {
                    atomicExch(status, kTimeoutEmpty);
                    ok = false;
                    break;
                }
                mbar_expect_tx(&full[s], kBytesA + kBytesB);
                tma_load_2d(smem_a + s * kBytesA, &map_a, &full[s], kb * kBlockK, m0);
                tma_load_2d(smem_b + s * kBytesB, &map_b, &full[s], kb * kBlockK, n0);
                issued = kb + 1;
            }
            if (!ok) {
                // let the copies already in flight land before the block gives up its shared memory
                for (int kb = max(0, issued - kStages); kb < issued; ++kb)
                    mbar_wait(&full[kb % kStages], (kb / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(kBlockM, BN);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % kStages;
                const uint32_t phase = (kb / kStages) & 1;
                if (!mbar_wait(&full[s], phase)) {
                    atomicExch(status, kTimeoutFull);
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
                    umma_bf16(tmem_base, a_desc, b_desc, idesc, (kb | k) != 0);
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(accum_full);
        }
    } else {
        // Epilogue: warp w may read the tensor-memory lanes 32 * (w % 4) .. + 31.
        const int quarter = warp & 3;
        const int a_row = m0 + quarter * 32 + lane;
        if (!mbar_wait(accum_full, 0)) {
            if (lane == 0) atomicExch(status, kTimeoutAccum);
        } else {
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                if (a_row >= rows_a) continue;
                if (!ep.swap) {
                    // C[a_row, n0 + c0 + j]
                    const size_t o = (size_t)a_row * ep.ldc + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int col = n0 + c0 + j;
                        if (col >= rows_b) break;
                        float v = __uint_as_float(r[j]);
                        if (ep.bias) v += ld_f(ep.bias, col, ep.bias_dt);
                        if (ep.accumulate) v += ld_f(ep.out, o + j, ep.out_dt);
                        st_f(ep.out, o + j, ep.out_dt, v);
                    }
                } else {
                    // C[n0 + c0 + j, a_row]: the lanes of a warp write neighbouring elements
                    const float b = ep.bias ? ld_f(ep.bias, a_row, ep.bias_dt) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tok = n0 + c0 + j;
                        if (tok >= rows_b) break;
                        const size_t o = (size_t)tok * ep.ldc + a_row;
                        float v = __uint_as_float(r[j]) + b;
                        if (ep.accumulate) v += ld_f(ep.out, o, ep.out_dt);
                        st_f(ep.out, o, ep.out_dt, v);
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

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

template <int BN, int kStages>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, int rows_a, int rows_b, int K, const EpilogueArgs& ep,
           int* status, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)kStages * (kBlockM * kBlockK * 2 + BN * kBlockK * 2) +
                            (2 * kStages + 1) * sizeof(uint64_t) + 16;
    static bool configured = false;
    if (!configured) {
        const cudaError_t e =
            cudaFuncSetAttribute(gemm_bf16_kernel<BN, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        NN_CHECK(e == cudaSuccess, "gemm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((rows_a + kBlockM - 1) / kBlockM, (rows_b + BN - 1) / BN);
    gemm_bf16_kernel<BN, kStages><<<grid, kThreads, smem, stream>>>(ma, mb, rows_a, rows_b, K, ep, status);
    NN_LAUNCH_OK("gemm_bf16");
    return 0;
}

}  // namespace

// Whether nncpu_linear_tc takes these sizes: both row strides must keep TMA's
// 16-byte rule, which for bfloat16 means multiples of 8 elements.
extern "C" int nncpu_linear_tc_supported(int M, int N, int K, int lda) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0;
}

// C[M, N] (+)= X[M, K] . W[N, K]^T + bias.  X and W are bfloat16; C is float or
// bfloat16 with row stride ldc; `status` is a device word that a kernel sets
// when one of its bounded waits ran out (the host checks it when it next
// synchronises).
extern "C" int nncpu_linear_tc(const void* X, const void* W, const void* bias, int bias_dt, void* C, int c_dt, int M,
                               int N, int K, int lda, int ldc, int accumulate, int* status, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(nncpu_linear_tc_supported(M, N, K, lda),
             "gemm: M %d, N %d, K %d, lda %d: K and lda must be multiples of 8 for the tensor-core path", M, N, K, lda);
    NN_CHECK(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm: operands must be 16-byte aligned");
    NN_CHECK(ldc >= N, "gemm: ldc %d is below N %d", ldc, N);
    EpilogueArgs ep{C, bias, c_dt, bias_dt, ldc, accumulate, 0};
    CUtensorMap ma, mb;
    if (M <= 256) {
        // few tokens: weights are the 128-row operand, tokens the narrow one
        ep.swap = 1;
        const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        if (int e = g_maps.get(&ma, W, N, K, K, kBlockM)) return e;
        if (int e = g_maps.get(&mb, X, M, K, lda, bn)) return e;
        switch (bn) {
            case 16: return launch<16, 8>(ma, mb, N, M, K, ep, status, stream);
            case 32: return launch<32, 8>(ma, mb, N, M, K, ep, status, stream);
            case 64: return launch<64, 8>(ma, mb, N, M, K, ep, status, stream);
            case 128: return launch<128, 6>(ma, mb, N, M, K, ep, status, stream);
            default: return launch<256, 4>(ma, mb, N, M, K, ep, status, stream);
        }
    }
    if (int e = g_maps.get(&ma, X, M, K, lda, kBlockM)) return e;
    if (N >= 256) {
        if (int e = g_maps.get(&mb, W, N, K, K, 256)) return e;
        return launch<256, 4>(ma, mb, M, N, K, ep, status, stream);
    }
    if (int e = g_maps.get(&mb, W, N, K, K, 128)) return e;
    return launch<128, 6>(ma, mb, M, N, K, ep, status, stream);
}
