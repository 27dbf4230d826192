// bfloat16 matrix product for very few tokens (at most 16):
//   C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias[N])      or      C[M, N/2] = silu(gate) * up
// With so few tokens the product is a stream over the weights and nothing
// else matters but keeping every SM's loads in flight: a block owns 16 weight
// rows, its eight warps each take an eighth of K, and every lane reads its
// rows 16 bytes at a time straight from global memory into the registers that
// feed mma.sync (m16n8k16: the 16 rows are weight rows, the 8 columns tokens).
// No shared-memory staging, no barriers in the stream, no scratch memory; the
// eight partial sums meet in shared memory and are added in warp order, so the
// result does not depend on timing.
//
// The 16 bytes a lane loads are 8 consecutive k of one row; the tensor core
// wants k pairs (2c, 2c+1, 2c+8, 2c+9) per lane.  Because a dot product does
// not care in which order k runs, weights and activations are simply loaded
// the same way and fed as if they were in the layout the instruction expects.
//
// The reference computes these products with its BF16 row kernels
// (crates/nncpu/src/kernels/mod.rs:337-360, crates/nncpu/src/kernels/scalar.rs:555-567).
//
// A decode step is a chain of these products with an RMS norm between every two of them, and at a few
// tokens such a norm is all launch and no work.  So the norm can ride on the products around it
// (y = (x * scale) * gamma with scale = 1 / sqrt(mean(x^2) + eps), crates/nncpu/src/kernels/scalar.rs:270-292):
//   * the product that adds into the residual stream ("producer") also writes x * gamma in bfloat16 for the
//     rows it has just finished, and adds the sum of squares of its 16 columns of every row to that row's total:
//     the blocks' sums meet in an exact accumulator per row: eight 64-bit integers, one per 32 binary orders of
//     magnitude, into which a float is added as its 24-bit mantissa shifted to its place.  Integer addition does
//     not care about order, so the blocks add with plain atomic adds that nobody waits for, and the total is the
//     same whatever the timing;
//   * the product that reads the normed rows ("consumer") takes x * gamma as its input, fetches the rows'
//     accumulators when it starts (72 bytes a row), turns them into the rows' scales after its weight stream, and
//     multiplies its own result by them, which a product commutes with.
// A producer also clears the accumulators of the norm before it, whose consumer has run by then.
//
// Two blocks of 8 warps run per SM.  A grid of N / 16 blocks that is a little more than that (N 5120: 320 blocks for
// 296 places) would leave its last blocks to stream alone, each at what one block can keep in flight; such a grid
// runs as blocks of 4 warps, four per SM, all at once with the same bytes in flight per SM.
//
// A step's products follow one another, and each would start with idle memory: launch, first addresses, the
// first bytes' way from memory.  So the kernel is launched to overlap with the end of the kernel before it
// (programmatic dependent launch): its blocks take the places that blocks of the earlier kernel leave, ask for
// their first weights, which depend on nobody, and only then wait for the earlier kernel's results.  Only after
// another product of this kind, though: a block that moves in beside blocks of a kernel with much shared memory
// (decode attention) keeps the SM in that kernel's split of shared memory and L1 for as long as the chain of
// overlapping products lasts, and with little L1 these products crawl (a decode layer took 135 us instead of 91).

#include <math.h>

#define NN_LIB linear_skinny
#define NN_LAUNCH_OVERLAP
#include "common.cuh"

namespace {

constexpr int kRows = 16;     // weight rows per block
constexpr int kUnroll = 8;    // 32-wide k groups in flight per warp with up to 8 tokens; 6 with up to 16 (registers)


enum Epilogue : int { kPlain = 0, kSwiglu = 1 };

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Weights are read once: stream them past the caches.
__device__ __forceinline__ uint4 ldg16_stream(const __nv_bfloat16* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ float silu_mul(float g, float u) { return (g * (1.0f / (1.0f + expf(0.0f - g)))) * u; }

// NT = number of 8-token tiles (1: up to 8 tokens, 2: up to 16); kW = warps of the block (8 or 4).
template <int NT, int kEpi, int kW>
__global__ void __launch_bounds__(kW * 32, 16 / kW)
skinny_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W, const void* __restrict__ bias,
              int bias_dt, void* __restrict__ out, int out_dt, int M, int N, int K, int lda, int ldc, int accumulate,
              const NormFusion nf) {
    constexpr int kU = NT == 1 ? kUnroll : 6;
    constexpr int kThreadsHere = kW * 32;
    constexpr int kPasses = kRows * 16 / kThreadsHere;   // output elements per thread: (token, row) pairs of 16 x 16
    __shared__ float part[kW][kRows][NT * 8 + 1];
    __shared__ float row_scale[16];
    __shared__ unsigned long long bins_s[16][9];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane & 3, r = lane >> 2;
    const int row0 = blockIdx.x * kRows;
    const int row_lo = row0 + r, row_hi = row0 + r + 8;
    const __nv_bfloat16* w_lo = W + (size_t)min(row_lo, N - 1) * K;
    const __nv_bfloat16* w_hi = W + (size_t)min(row_hi, N - 1) * K;
    const __nv_bfloat16* x0 = X + (size_t)min(r, M - 1) * lda;
    const __nv_bfloat16* x1 = X + (size_t)min(r + 8, M - 1) * lda;

    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;

    // this warp's share of K, in groups of 32
    const int n_groups = (K + 31) / 32;
    const int per_warp = (n_groups + kW - 1) / kW;
    const int g_begin = warp * per_warp, g_end = min(n_groups, g_begin + per_warp);
    // Full blocks of kUnroll groups: every load is issued before the first product, without predicates.
    // Columns of tokens beyond M read a valid row and are never stored.
    const int k_full = K / 32;                        // groups that lie wholly inside K
    const int g_fast_end = min(g_end, k_full);

    // The first weights are asked for before anything that an earlier kernel may still be writing is touched.
    let_next_kernel_start();
    uint4 a_lo[kU], a_hi[kU];
    if (g_begin + kU <= g_fast_end) {
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int k = (g_begin + u) * 32 + c * 8;
            a_lo[u] = ldg16_stream(w_lo + k);
            a_hi[u] = ldg16_stream(w_hi + k);
        }
    }
    wait_for_previous_kernels();

    // What the product is added to is fetched now, under the weight stream, not after it: thread i of the
    // epilogue owns output (token i / 16, row i % 16); with at most 16 tokens that is one element per thread.
    float before[kPasses];
#pragma unroll
    for (int e = 0; e < kPasses; ++e) {
        before[e] = 0.0f;
        if (kEpi == kPlain && accumulate) {
            const int i = threadIdx.x + e * kThreadsHere;
            const int tok = i / kRows, row = row0 + i % kRows;
            if (tok < M && row < N) before[e] = ld_f(out, (size_t)tok * ldc + row, out_dt);
        }
    }

    // Consumer of a norm: the rows' accumulators are asked for now (asynchronous 8-byte copies into shared memory
    // that hold no register and stall nobody) and turned into scales after the weight stream.
    if (nf.bins_in != nullptr && threadIdx.x < M) {
        // thread t fetches row t's accumulator for itself: when its own copies have landed it needs nobody else
#pragma unroll
        for (int word = 0; word < 9; ++word)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(&bins_s[threadIdx.x][word])),
                         "l"(nf.bins_in + threadIdx.x * kBinWords + word)
                         : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // Producer of a norm: the accumulators of the norm before it are cleared for their next use.
    if (nf.bins_clear != nullptr && blockIdx.x == 0)
        for (int i = threadIdx.x; i < 16 * kBinWords; i += kThreadsHere) nf.bins_clear[i] = 0ull;

    int g0 = g_begin;
    for (; g0 + kU <= g_fast_end; g0 += kU) {
        uint4 b0[kU], b1[kU];
        if (g0 != g_begin) {
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int k = (g0 + u) * 32 + c * 8;
                a_lo[u] = ldg16_stream(w_lo + k);
                a_hi[u] = ldg16_stream(w_hi + k);
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int k = (g0 + u) * 32 + c * 8;
            b0[u] = *reinterpret_cast<const uint4*>(x0 + k);
            if (NT > 1) b1[u] = *reinterpret_cast<const uint4*>(x1 + k);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            mma_bf16(acc[0], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b0[u].x, b0[u].y);
            mma_bf16(acc[0], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b0[u].z, b0[u].w);
            if (NT > 1) {
                mma_bf16(acc[1], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b1[u].x, b1[u].y);
                mma_bf16(acc[1], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b1[u].z, b1[u].w);
            }
        }
    }
    // The rest (fewer than a full round of groups, the last of them perhaps cut by K) as one more round whose loads
    // are all issued before the first product, with zeros where there is nothing: K is a multiple of 8, so a
    // 16-byte chunk is inside K or outside.
    if (g0 < g_end) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        uint4 b0[kU], b1[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int k = (g0 + u) * 32 + c * 8;
            const bool ok = g0 + u < g_end && k < K;
            a_lo[u] = ok ? ldg16_stream(w_lo + k) : z;
            a_hi[u] = ok ? ldg16_stream(w_hi + k) : z;
            b0[u] = ok ? *reinterpret_cast<const uint4*>(x0 + k) : z;
            if (NT > 1) b1[u] = ok ? *reinterpret_cast<const uint4*>(x1 + k) : z;
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            mma_bf16(acc[0], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b0[u].x, b0[u].y);
            mma_bf16(acc[0], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b0[u].z, b0[u].w);
            if (NT > 1) {
                mma_bf16(acc[1], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b1[u].x, b1[u].y);
                mma_bf16(acc[1], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b1[u].z, b1[u].w);
            }
        }
    }
    // accumulator layout: [0..1] row r, tokens 2c, 2c+1; [2..3] row r + 8
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        part[warp][r][t * 8 + 2 * c] = acc[t][0];
        part[warp][r][t * 8 + 2 * c + 1] = acc[t][1];
        part[warp][r + 8][t * 8 + 2 * c] = acc[t][2];
        part[warp][r + 8][t * 8 + 2 * c + 1] = acc[t][3];
    }
    if (nf.bins_in != nullptr && threadIdx.x < M) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        row_scale[threadIdx.x] = 1.0f / sqrtf(bins_total(bins_s[threadIdx.x]) * (1.0f / (float)K) + nf.eps);
    }
    __syncthreads();
    if (kEpi == kSwiglu) {
        // rows 0..7 of the block are gate rows, rows 8..15 the up rows of the same outputs
        for (int i = threadIdx.x; i < 8 * M; i += kThreadsHere) {
            const int tok = i / 8, j = i % 8;
            if (row0 + j + 8 >= N) continue;
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int w = 0; w < kW; ++w) {
                g += part[w][j][tok];
                u += part[w][j + 8][tok];
            }
            if (nf.bins_in != nullptr) {
                g *= row_scale[tok];
                u *= row_scale[tok];
            }
            st_f(out, (size_t)tok * ldc + (row0 >> 1) + j, out_dt, silu_mul(g, u));
        }
    } else {
        // output element i is (token i / 16, row i % 16): one per thread of 8 warps, two per thread of 4; every thread
        // of the block walks through (the producer's sums of squares are taken with shuffles)
#pragma unroll
        for (int e = 0; e < kPasses; ++e) {
            const int i = threadIdx.x + e * kThreadsHere;
            const int tok = i / kRows, j = i % kRows;
            const int row = row0 + j;
            const bool valid = tok < M && row < N;
            float v = 0.0f;
            if (valid) {
#pragma unroll
                for (int w = 0; w < kW; ++w) v += part[w][j][tok];
                if (nf.bins_in != nullptr) v *= row_scale[tok];
                if (bias) v += ld_f(bias, row, bias_dt);
                if (accumulate) v += before[e];
                st_f(out, (size_t)tok * ldc + row, out_dt, v);
            }
            if (nf.xg_out != nullptr) {
                // producer of a norm: x * gamma for the consumer, and this block's part of every row's sum of squares
                // (the 16 lanes that hold a row's 16 columns add up through the shuffle tree)
                if (valid) nf.xg_out[(size_t)tok * N + row] = __float2bfloat16(v * ld_f(nf.gamma, row, nf.gamma_dt));
                float sq = valid ? v * v : 0.0f;
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (j == 0 && tok < M) bins_add(nf.bins_out + tok * kBinWords, sq);
            }
        }
    }
}

int sm_count() {
    static int counts[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (counts[dev] == 0 && cudaDeviceGetAttribute(&counts[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        counts[dev] = 148;
    return counts[dev];
}

// Blocks of 4 warps (four per SM) or of 8 (two per SM)?  What a product costs beyond its bytes are the round trips
// to memory that follow one another: a warp makes one per round of `unroll` groups of its share of K, and a grid
// makes one pass per filling of the SMs' places.  The smaller count of (passes x rounds) wins; on a tie the
// small blocks, if the big ones would leave a nearly empty second pass (at most four blocks per SM) or with two
// token tiles.  Measured on the layer shapes and output matrices of the 8B, 14B and 32B sizes at 8 and 16 tokens
// (26 cases, differences of 3 to 30 %): the rule picks the faster kind in all of them.
bool four_warps_pay(int blocks, int K, int unroll, int sms) {
    const int groups = (K + 31) / 32;
    auto cost = [&](int warps) {
        const int places = (16 / warps) * sms;
        const int passes = (blocks + places - 1) / places;
        const int per_warp = (groups + warps - 1) / warps;
        return (long)passes * ((per_warp + unroll - 1) / unroll);
    };
    const long big = cost(8), small = cost(4);
    if (small != big) return small < big;
    return blocks > 2 * sms && (blocks <= 4 * sms || unroll < kUnroll);
}

int g_forced_warps = 0;   // measurements and tests: blocks of 8 or of 4 warps whatever the sizes (0: by the sizes)

template <int NT, int kEpi>
int launch(const void* X, const void* W, const void* bias, int bias_dt, void* C, int c_dt, int M, int N, int K, int lda,
           int ldc, int accumulate, const NormFusion& nf, bool overlap, cudaStream_t stream) {
    const int blocks = (N + kRows - 1) / kRows;
    const bool small = g_forced_warps ? g_forced_warps == 4 : four_warps_pay(blocks, K, NT == 1 ? kUnroll : 6, sm_count());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(small ? 128 : 256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    cfg.numAttrs = overlap ? overlap_attribute(attr) : 0;
    cfg.attrs = attr;
    const cudaError_t e =
        small ? cudaLaunchKernelEx(&cfg, skinny_kernel<NT, kEpi, 4>, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, bias,
                                   bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf)
              : cudaLaunchKernelEx(&cfg, skinny_kernel<NT, kEpi, 8>, (const __nv_bfloat16*)X, (const __nv_bfloat16*)W, bias,
                                   bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf);
    NN_CHECK(e == cudaSuccess, "linear (few tokens): launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

// For measurements and tests: blocks of 8 or of 4 warps whatever the sizes; 0: chosen by the sizes.
extern "C" void nncpu_linear_skinny_force_warps(int warps) { g_forced_warps = warps; }

extern "C" int nncpu_linear_skinny_supported(int M, int N, int K, int lda) {
    return M > 0 && M <= 16 && N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0;
}

// 64-bit words of the accumulators of one norm (16 rows): what a producer adds into and a consumer reads.
extern "C" int nncpu_linear_skinny_norm_words() { return 16 * kBinWords; }

// C[M, N] (+)= X[M, K] . W[N, K]^T + bias for M <= 16, or with epilogue 1: C[M, N/2] = silu(gate) * up
// for W rows interleaved in blocks of 8.  X and W are bfloat16 and 16-byte aligned; C is float or bfloat16.
//
// Norm fusion (see the head of this file), all optional; an accumulator block is nncpu_linear_skinny_norm_words()
// 64-bit words:
//   producer (plain epilogue): xg_out bfloat16 [M, N] receives C * gamma (gamma: N weights of type gamma_dt) and
//     bins_out, which must be zero, the sums of squares of C's rows; bins_clear (may be null) is set to zero;
//   consumer: X holds such C * gamma rows of width K and bins_in their accumulators: the result is multiplied by
//     1 / sqrt(sum / K + eps) per row before bias and activation.
// after_skinny: the kernel before this one in the stream is a product of this function too; then this one may start
// while that one ends (switched off for the whole library by nncpu_launch_overlap_linear_skinny(0)).
extern "C" int nncpu_linear_skinny(const void* X, const void* W, const void* bias, int bias_dt, void* C, int c_dt,
                                   int M, int N, int K, int lda, int ldc, int accumulate, int epilogue, void* xg_out,
                                   const void* gamma, int gamma_dt, void* bins_out, void* bins_clear,
                                   const void* bins_in, float eps, int after_skinny, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(nncpu_linear_skinny_supported(M, N, K, lda),
             "linear (few tokens): M %d, N %d, K %d, lda %d: at most 16 tokens, K and lda multiples of 8", M, N, K, lda);
    NN_CHECK(((uintptr_t)X % 16) == 0 && ((uintptr_t)W % 16) == 0, "linear (few tokens): operands must be 16-byte aligned");
    NN_CHECK(epilogue == kPlain || epilogue == kSwiglu, "linear (few tokens): unknown epilogue %d", epilogue);
    const int n_out = epilogue == kSwiglu ? N / 2 : N;
    NN_CHECK(ldc >= n_out, "linear (few tokens): ldc %d is below the %d output features", ldc, n_out);
    NormFusion nf{};
    if (xg_out != nullptr) {
        NN_CHECK(epilogue == kPlain && gamma != nullptr && bins_out != nullptr && ((uintptr_t)bins_out % 8) == 0 &&
                     ((uintptr_t)bins_clear % 8) == 0,
                 "linear (few tokens): leaving a norm's input needs the plain epilogue, the norm's weights and its "
                 "accumulators (8-byte aligned)");
        nf.xg_out = (__nv_bfloat16*)xg_out;
        nf.gamma = gamma;
        nf.gamma_dt = gamma_dt;
        nf.bins_out = (unsigned long long*)bins_out;
        nf.bins_clear = (unsigned long long*)bins_clear;
    }
    if (bins_in != nullptr) {
        NN_CHECK(((uintptr_t)bins_in % 8) == 0 && eps >= 0.0f, "linear (few tokens): a norm's accumulators (8-byte aligned), eps %g",
                 eps);
        nf.bins_in = (const unsigned long long*)bins_in;
        nf.eps = eps;
    }
    if (epilogue == kSwiglu) {
        NN_CHECK(N % 16 == 0 && bias == nullptr && !accumulate,
                 "linear (few tokens): the gated epilogue needs N %% 16 == 0, no bias and no accumulation (N %d)", N);
        return M <= 8 ? launch<1, kSwiglu>(X, W, bias, bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf, after_skinny != 0, stream)
                      : launch<2, kSwiglu>(X, W, bias, bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf, after_skinny != 0, stream);
    }
    return M <= 8 ? launch<1, kPlain>(X, W, bias, bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf, after_skinny != 0, stream)
                  : launch<2, kPlain>(X, W, bias, bias_dt, C, c_dt, M, N, K, lda, ldc, accumulate, nf, after_skinny != 0, stream);
}
