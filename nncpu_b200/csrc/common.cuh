// Shared helpers of the sm_100a kernels: element-type codes, loads and stores
// that widen to float, block reductions, and the error channel of the C entry
// points.  Every entry point returns 0 on success; on refusal it returns a
// non-zero code and leaves a message for nncpu_last_error().
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

enum DType : int { DT_F32 = 0, DT_BF16 = 1 };

constexpr int kPage = 64;  // tokens per cache page; the host-side cache uses the same number

// Each library built from these sources keeps its own message; NN_LIB names the
// library and the exported function that returns the message.
#ifndef NN_LIB
#error "define NN_LIB (the library's name) before including common.cuh"
#endif
#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

static void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

#define NN_CAT2(a, b) a##b
#define NN_CAT(a, b) NN_CAT2(a, b)
extern "C" const char* NN_CAT(nncpu_last_error_, NN_LIB)() { return g_error; }

#define NN_CHECK(cond, ...)            \
    do {                               \
        if (!(cond)) {                 \
            set_error(__VA_ARGS__);    \
            return 1;                  \
        }                              \
    } while (0)

#define NN_LAUNCH_OK(name)                                                        \
    do {                                                                          \
        cudaError_t e_ = cudaGetLastError();                                      \
        if (e_ != cudaSuccess) {                                                  \
            set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));     \
            return 2;                                                             \
        }                                                                         \
    } while (0)

__device__ __forceinline__ float ld_f(const void* p, size_t i, int dt) {
    return dt == DT_F32 ? reinterpret_cast<const float*>(p)[i]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void st_f(void* p, size_t i, int dt, float v) {
    if (dt == DT_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// True the first time a call site asks on the current device: for set-up that belongs to a (kernel, device)
// pair, such as the shared-memory attribute.  `done` is the call site's own static array.
inline bool first_use_on_this_device(bool (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done[dev]) return false;
    done[dev] = true;
    return true;
}

// Programmatic dependent launch: a kernel launched with `overlap_attribute` may start while the kernel before it in
// the stream still runs, once every block of that kernel has called let_next_kernel_start() (or has ended).  It
// may do only what does not depend on earlier kernels (fetch weights) until wait_for_previous_kernels() returns:
// from then on everything that earlier kernels wrote is visible and nothing of them still runs.  Every kernel that is
// launched with the attribute calls both; without the attribute both do nothing.  A library that uses this defines
// NN_LAUNCH_OVERLAP before it includes this file and exports nncpu_launch_overlap_<library>(on) (default: on).
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_previous_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

#ifdef NN_LAUNCH_OVERLAP
static bool g_launch_overlap = true;
extern "C" void NN_CAT(nncpu_launch_overlap_, NN_LIB)(int on) { g_launch_overlap = on != 0; }
// Fills `attr` and returns how many attributes to pass on (0 when the overlap is switched off).
inline unsigned overlap_attribute(cudaLaunchAttribute* attr) {
    attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr->val.programmaticStreamSerializationAllowed = 1;
    return g_launch_overlap ? 1u : 0u;
}
#endif

// ---------------------------------------------------------------------------
// Norms that ride on the products around them (linear_skinny.cu explains the scheme; the tensor-core products of
// whole prompts do the same).  A row's sum of squares is kept in an exact accumulator of kBinWords 64-bit words:
// eight integers, one per 32 binary orders of magnitude, a word that counts values that are not finite, and spare
// words that keep a row at 128 bytes.
// ---------------------------------------------------------------------------
// What a product does for the norms around it (all null or zero: nothing).
constexpr int kBinWords = 16;    // 64-bit words a row: 8 accumulator bins, a word that says "not finite", 7 spare
struct NormFusion {
    // producer: besides C, leave the input of the norm that reads C next
    __nv_bfloat16* xg_out;        // [M, N]: C * gamma, not yet multiplied by the row's scale
    const void* gamma;            // [N] weights of that norm
    int gamma_dt;
    unsigned long long* bins_out; // [rows, kBinWords], zero before the launch: the rows' sums of squares of C
    unsigned long long* bins_clear;  // [rows, kBinWords] of an earlier norm whose consumer has run: set to zero (or null)
    // consumer: X is such an input; the rows' scales are applied to this product's result
    const unsigned long long* bins_in;   // [rows, kBinWords]
    float eps;
};

// A non-negative float into its row's accumulator: value = mantissa * 2^(E - 150) with E = 32 * bin + shift.
__device__ __forceinline__ void bins_add(unsigned long long* bins, float v) {
    const uint32_t bits = __float_as_uint(v);
    const uint32_t e = (bits >> 23) & 0xFF;
    if (e == 0xFF) {                       // infinity or NaN: the row has no finite norm
        atomicAdd(bins + 8, 1ull);
        return;
    }
    const uint32_t ee = e ? e : 1;         // subnormals have the exponent of the smallest normal and no hidden bit
    const unsigned long long mant = (bits & 0x7FFFFF) | (e ? 0x800000u : 0u);
    if (mant) atomicAdd(bins + ee / 32, mant << (ee % 32));
}

// The sum that an accumulator holds, as a float: every bin is rounded to float and weighted with its power of two
// (2^(32 b - 150), applied as two factors of 2^(16 b - 75) so that neither leaves the float range), and the eight
// terms are added in bin order.  Eight roundings of 2^-24: the accumulators are exact so that the sum does not depend
// on the order in which blocks add to it, not because its last bits matter (the norm's own kernel adds 4 096 squares
// in float).  The terms do not depend on one another, which keeps this short where it stands at the end of a block:
// an exact conversion in 64-bit floating point or in 128-bit integers cost a decode step's consumers twice as much.
__device__ __forceinline__ float bins_total(const unsigned long long* bins) {
    if (bins[8] != 0) return __int_as_float(0x7FC00000);   // NaN
    float s = 0.0f;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        const float c = __int_as_float((127 + 16 * b - 75) << 23);   // 2^(16 b - 75)
        s += (__ull2float_rn(bins[b]) * c) * c;
    }
    return s;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats.  The order of additions is fixed, so the result
// does not depend on anything but the inputs.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
