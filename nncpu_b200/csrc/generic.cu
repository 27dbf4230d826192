// Kernels that take every size and both element types (float and bfloat16,
// chosen per tensor at run time) and compute in 32-bit: the whole float32 path
// of the model runs on them, and the bfloat16 path uses them wherever no
// specialised kernel applies.  Plain CUDA cores, no reduced-precision matrix
// mode anywhere in this file.
//
// The arithmetic follows ZacWalk/nncpu's scalar kernels:
//   RMSNorm            crates/nncpu/src/kernels/scalar.rs:270-292
//   rotary embedding   crates/nncpu/src/kernels/mod.rs:687-737
//   attention          crates/nncpu/src/kernels/scalar.rs:444-548 (online softmax, scale after the dot)
//   SiLU gate          crates/nncpu/src/kernels/scalar.rs:102-106,146-150
//   argmax             crates/nncpu/src/model/forward.rs:1003-1011 (first largest)
//   temperature draw   crates/nncpu/src/session/sample.rs:186-200

#include <math.h>

#define NN_LIB generic
#define NN_LAUNCH_OVERLAP
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding rows: out[t, :] = table[ids[t], :] * scale, float32 out.
// A negative id (a padded row) gives zeros.
// ---------------------------------------------------------------------------
__global__ void embed_kernel(const void* __restrict__ table, int table_dt, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[(size_t)t * hidden + i] = id < 0 ? 0.0f : ld_f(table, (size_t)id * hidden + i, table_dt) * scale;
}

extern "C" int nncpu_embed(const void* table, int table_dt, const int* ids, float* out, int n_tok, int hidden,
                           int vocab, float scale, void* stream) {
    NN_CHECK(n_tok >= 0 && hidden > 0 && vocab > 0, "embed: n_tok %d, hidden %d, vocab %d", n_tok, hidden, vocab);
    if (n_tok == 0) return 0;
    embed_kernel<<<n_tok, 256, 0, (cudaStream_t)stream>>>(table, table_dt, ids, out, hidden, scale);
    NN_LAUNCH_OK("embed");
    return 0;
}

// ---------------------------------------------------------------------------
// RMSNorm over the last axis: y = (x * scale) * gamma,
// scale = 1 / sqrt(mean(x^2) + eps).  `rows` (optional) picks input rows, so
// the final norm runs only on the rows whose logits are wanted.
// ---------------------------------------------------------------------------
__global__ void rmsnorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ gamma, int g_dt,
                               void* __restrict__ y, int y_dt, const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    if (r_in < 0) {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) st_f(y, (size_t)r_out * dim + i, y_dt, 0.0f);
        return;
    }
    const size_t base = (size_t)r_in * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = ld_f(x, base + i, x_dt);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss * (1.0f / (float)dim) + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = ld_f(x, base + i, x_dt) * scale;
        st_f(y, (size_t)r_out * dim + i, y_dt, gamma ? v * ld_f(gamma, i, g_dt) : v);
    }
}

// The common case, float32 rows of a width that is a multiple of 4 and at most 256 * 4 * kVec: every
// thread keeps its part of the row in registers between the sum of squares and the scaling, so the
// row is read once, 16 bytes at a time.
template <int kVec>
__global__ void __launch_bounds__(256)
rmsnorm_f32_kernel(const float* __restrict__ x, const void* __restrict__ gamma, int g_dt, void* __restrict__ y,
                   int y_dt, const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    // launched to start while the kernel before it ends: the product that follows may set itself up meanwhile
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    const int n4 = dim >> 2;
    float4 v[kVec];
    float ss = 0.0f;
    if (r_in >= 0) {
        const float4* src = reinterpret_cast<const float4*>(x + (size_t)r_in * dim);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < n4 ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    ss = block_sum(ss, scratch);
    const float scale = r_in >= 0 ? 1.0f / sqrtf(ss * (1.0f / (float)dim) + eps) : 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float o[4] = {v[j].x * scale, v[j].y * scale, v[j].z * scale, v[j].w * scale};
        if (gamma) {
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] *= ld_f(gamma, 4 * i + e, g_dt);
        }
        const size_t at = (size_t)r_out * dim + 4 * i;
        if (y_dt == DT_BF16) {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + at) = *reinterpret_cast<uint2*>(h);
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + at) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

extern "C" int nncpu_rmsnorm(const void* x, int x_dt, const void* gamma, int g_dt, void* y, int y_dt,
                             const int* rows, int n_rows, int dim, float eps, void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "rmsnorm: %d rows of %d", n_rows, dim);
    if (n_rows == 0) return 0;
    if (x_dt == DT_F32 && dim % 4 == 0 && dim >= 1024 && dim <= 256 * 4 * 8 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)y % 16 == 0) {
        const float* xf = (const float*)x;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_rows);
        cfg.blockDim = dim3(256);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        cfg.attrs = attr;
        cfg.numAttrs = overlap_attribute(attr);
        const auto kernel = dim <= 256 * 4 * 2 ? rmsnorm_f32_kernel<2> : dim <= 256 * 4 * 4 ? rmsnorm_f32_kernel<4> : rmsnorm_f32_kernel<8>;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, xf, gamma, g_dt, y, y_dt, rows, dim, eps);
        NN_CHECK(e == cudaSuccess, "rmsnorm: launch failed: %s", cudaGetErrorString(e));
        return 0;
    }
    int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : (dim >= 128 ? 128 : 32));
    rmsnorm_kernel<<<n_rows, threads, 0, (cudaStream_t)stream>>>(x, x_dt, gamma, g_dt, y, y_dt, rows, dim, eps);
    NN_LAUNCH_OK("rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------
// C[M, N] (+)= A[M, K] . W[N, K]^T + bias[N], 32-bit multiply-add on CUDA
// cores.  Each output element is summed over k in ascending order by one
// thread, so a row's result does not depend on which other rows are present.
// ---------------------------------------------------------------------------
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
linear_simt_kernel(const void* __restrict__ A, int a_dt, const void* __restrict__ W, int w_dt,
                   const void* __restrict__ bias, int b_dt, void* __restrict__ C, int c_dt, int M, int N, int K,
                   int lda, int ldc, int accumulate) {
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int m = m0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? ld_f(A, (size_t)m * lda + k, a_dt) : 0.0f;
        }
        for (int e = tid; e < BN * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int n = n0 + r, k = k0 + c;
            Ws[c][r] = (n < N && k < K) ? ld_f(W, (size_t)n * K + k, w_dt) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += ld_f(bias, n, b_dt);
            const size_t o = (size_t)m * ldc + n;
            if (accumulate) v += ld_f(C, o, c_dt);
            st_f(C, o, c_dt, v);
        }
    }
}

extern "C" int nncpu_linear_simt(const void* A, int a_dt, const void* W, int w_dt, const void* bias, int b_dt,
                                 void* C, int c_dt, int M, int N, int K, int lda, int ldc, int accumulate,
                                 void* stream) {
    NN_CHECK(M >= 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "linear: M %d, N %d, K %d, lda %d, ldc %d", M, N,
             K, lda, ldc);
    if (M == 0) return 0;
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16);
        linear_simt_kernel<16, 64, 32, 2, 2><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, bias, b_dt, C, c_dt, M, N, K, lda, ldc, accumulate);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        linear_simt_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, bias, b_dt, C, c_dt, M, N, K, lda, ldc, accumulate);
    }
    NN_LAUNCH_OK("linear");
    return 0;
}

// ---------------------------------------------------------------------------
// Rotation table of a step: cs[t, i] = (cos, sin)(float(pos_t) * pos_scale * inv_freq[i]), or with
// by_pair the same values laid out [i, t] for readers whose lanes are tokens.
// Computed once per step and read by every layer that shares the encoding.
// ---------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int n_tok, int half, float pos_scale, int by_pair) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * half) return;
    const int t = by_pair ? idx % n_tok : idx / half, i = by_pair ? idx / n_tok : idx % half;
    const float theta = ((float)pos[t] * pos_scale) * inv_freq[i];
    float s, c;
    sincosf(theta, &s, &c);
    cs[idx] = make_float2(c, s);
}

extern "C" int nncpu_rope_table(const int* pos, const float* inv_freq, float* cs, int n_tok, int half,
                                float pos_scale, int by_pair, void* stream) {
    NN_CHECK(n_tok >= 0 && half > 0, "rope_table: %d tokens, %d pairs", n_tok, half);
    if (n_tok == 0) return 0;
    const int total = n_tok * half;
    NN_CHECK((uintptr_t)cs % 8 == 0, "rope_table: the table must be 8-byte aligned (it is written as cos/sin pairs)");
    rope_table_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(pos, inv_freq, (float2*)cs, n_tok,
                                                                             half, pos_scale, by_pair);
    NN_LAUNCH_OK("rope_table");
    return 0;
}

// ---------------------------------------------------------------------------
// Per-head q/k RMSNorm, rotation, and the append of k and v to the cache.
// qkv [n_tok, (n_heads + 2 n_kv) * hd] holds q heads, then k heads, then v
// heads.  One warp per (token, head).  q goes to q_out [n_tok, n_heads * hd];
// k (normed, rotated) and v (raw) go to their page rows.  With n_kv == 0 the
// mixer reads another layer's cache and only q is processed.
// ---------------------------------------------------------------------------
__global__ void qk_norm_rope_append_kernel(const void* __restrict__ qkv, int in_dt, const void* __restrict__ q_gamma,
                                           const void* __restrict__ k_gamma, int g_dt, float eps,
                                           const float2* __restrict__ cs, int rot_half,
                                           const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                           const int* __restrict__ block_table, int bt_stride,
                                           void* __restrict__ k_pages, void* __restrict__ v_pages, int kv_dt,
                                           void* __restrict__ q_out, int q_dt, int n_tok, int n_heads, int n_kv,
                                           int hd) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = n_heads + 2 * n_kv;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long)n_tok * per_tok) return;
    const int t = (int)(item / per_tok), h = (int)(item % per_tok);
    const int seq = tok_seq[t];
    float* x = smem + warp * hd;
    const size_t in_base = (size_t)t * per_tok * hd + (size_t)h * hd;
    const bool is_q = h < n_heads, is_k = !is_q && h < n_heads + n_kv;
    const void* gamma = is_q ? q_gamma : (is_k ? k_gamma : nullptr);

    float ss = 0.0f;
    for (int i = lane; i < hd; i += 32) {
        const float v = ld_f(qkv, in_base + i, in_dt);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (gamma) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)hd) + eps);
        for (int i = lane; i < hd; i += 32) x[i] = (x[i] * scale) * ld_f(gamma, i, g_dt);
    }
    __syncwarp();
    if ((is_q || is_k) && cs != nullptr) {
        for (int i = lane; i < rot_half; i += 32) {
            const float2 c = cs[(size_t)t * rot_half + i];
            const float a = x[i], b = x[i + rot_half];
            x[i] = c.x * a - c.y * b;
            x[i + rot_half] = c.y * a + c.x * b;
        }
        __syncwarp();
    }
    if (is_q) {
        const size_t o = (size_t)t * n_heads * hd + (size_t)h * hd;
        for (int i = lane; i < hd; i += 32) st_f(q_out, o + i, q_dt, x[i]);
        return;
    }
    if (seq < 0) return;  // a padded row owns no place in the cache
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)seq * bt_stride + pos / kPage];
    if (page < 0) return;
    const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
    const size_t o = (((size_t)page * n_kv + kvh) * kPage + pos % kPage) * hd;
    void* dst = is_k ? k_pages : v_pages;
    for (int i = lane; i < hd; i += 32) st_f(dst, o + i, kv_dt, x[i]);
}

// The bfloat16 run's case: float32 projections in, bfloat16 q and cache out, the whole head rotated,
// head size 64 or 128.  A lane holds EPL = hd / 32 neighbouring lanes of the head, so lanes 0-15 hold
// the first half and lanes 16-31 the second: a rotation pair sits in lanes i and i + 16.
template <int EPL>
__global__ void __launch_bounds__(256)
qk_norm_rope_append_fast_kernel(const float* __restrict__ qkv, const void* __restrict__ q_gamma,
                                const void* __restrict__ k_gamma, int g_dt, float eps, const float2* __restrict__ cs,
                                const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                                __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ q_out, int n_tok,
                                int n_heads, int n_kv) {
    constexpr int hd = 32 * EPL, half = hd / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = n_heads + 2 * n_kv;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= (long)n_tok * per_tok) return;
    const int t = (int)(item / per_tok), h = (int)(item % per_tok);
    const bool is_q = h < n_heads, is_k = !is_q && h < n_heads + n_kv;
    const float* src = qkv + ((size_t)t * per_tok + h) * hd + lane * EPL;
    float x[EPL];
    if (EPL == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        x[0] = v.x; x[1] = v.y; x[2 % EPL] = v.z; x[3 % EPL] = v.w;
    } else {
        const float2 v = *reinterpret_cast<const float2*>(src);
        x[0] = v.x; x[1] = v.y;
    }
    const void* gamma = is_q ? q_gamma : (is_k ? k_gamma : nullptr);
    if (gamma) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) ss = fmaf(x[e], x[e], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)hd) + eps);
#pragma unroll
        for (int e = 0; e < EPL; ++e) x[e] = (x[e] * scale) * ld_f(gamma, lane * EPL + e, g_dt);
    }
    if ((is_q || is_k) && cs != nullptr) {
        const int i0 = (lane & 15) * EPL;   // index of the rotation pair
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            const float2 c = cs[(size_t)t * half + i0 + e];
            x[e] = lane < 16 ? c.x * x[e] - c.y * other : c.y * other + c.x * x[e];
        }
    }
    __nv_bfloat16* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * n_heads + h) * hd;
    } else {
        const int seq = tok_seq[t];
        if (seq < 0) return;
        const int pos = tok_pos[t];
        const int page = block_table[(size_t)seq * bt_stride + pos / kPage];
        if (page < 0) return;
        const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
        dst = (is_k ? k_pages : v_pages) + (((size_t)page * n_kv + kvh) * kPage + pos % kPage) * hd;
    }
    if (EPL == 4) {
        __nv_bfloat162 o[2] = {__floats2bfloat162_rn(x[0], x[1]), __floats2bfloat162_rn(x[2 % EPL], x[3 % EPL])};
        *reinterpret_cast<uint2*>(dst + lane * 4) = *reinterpret_cast<uint2*>(o);
    } else {
        *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(x[0], x[1]);
    }
}

extern "C" int nncpu_qk_norm_rope_append(const void* qkv, int in_dt, const void* q_gamma, const void* k_gamma,
                                         int g_dt, float eps, const float* cs, int rot_half, const int* tok_seq,
                                         const int* tok_pos, const int* block_table, int bt_stride, void* k_pages,
                                         void* v_pages, int kv_dt, void* q_out, int q_dt, int n_tok, int n_heads,
                                         int n_kv, int hd, void* stream) {
    NN_CHECK(n_tok >= 0 && n_heads > 0 && n_kv >= 0 && hd > 0, "qk_norm_rope_append: sizes");
    NN_CHECK(hd % 2 == 0 && 2 * rot_half <= hd, "qk_norm_rope_append: head size %d with %d rotated pairs", hd,
             rot_half);
    NN_CHECK((uintptr_t)cs % 8 == 0, "qk_norm_rope_append: the rotation table must be 8-byte aligned (cos/sin pairs)");
    NN_CHECK(hd <= 1024, "qk_norm_rope_append: head size %d is above 1024", hd);
    if (n_tok == 0) return 0;
    if (in_dt == DT_F32 && q_dt == DT_BF16 && (n_kv == 0 || kv_dt == DT_BF16) && (hd == 64 || hd == 128) &&
        (cs == nullptr || 2 * rot_half == hd) && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0) {
        const long n_items = (long)n_tok * (n_heads + 2 * n_kv);
        const unsigned n_blocks = (unsigned)((n_items + 7) / 8);
        if (hd == 128)
            qk_norm_rope_append_fast_kernel<4><<<n_blocks, 256, 0, (cudaStream_t)stream>>>(
                (const float*)qkv, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, tok_seq, tok_pos, block_table,
                bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_tok, n_heads, n_kv);
        else
            qk_norm_rope_append_fast_kernel<2><<<n_blocks, 256, 0, (cudaStream_t)stream>>>(
                (const float*)qkv, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, tok_seq, tok_pos, block_table,
                bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_tok, n_heads, n_kv);
        NN_LAUNCH_OK("qk_norm_rope_append");
        return 0;
    }
    const int warps = 4;
    const long items = (long)n_tok * (n_heads + 2 * n_kv);
    const long blocks = (items + warps - 1) / warps;
    qk_norm_rope_append_kernel<<<(unsigned)blocks, warps * 32, warps * hd * sizeof(float), (cudaStream_t)stream>>>(
        qkv, in_dt, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, rot_half, tok_seq, tok_pos, block_table,
        bt_stride, k_pages, v_pages, kv_dt, q_out, q_dt, n_tok, n_heads, n_kv, hd);
    NN_LAUNCH_OK("qk_norm_rope_append");
    return 0;
}

// ---------------------------------------------------------------------------
// Attention of every (token, head) over the cache of the token's sequence:
// keys first..pos with first = max(0, pos + 1 - window) (window 0: all).
// One block per (token, head) walks the span in chunks of 128 keys with an
// online softmax; the chunk boundaries are fixed by the span alone, so the
// result does not depend on the batch or on how tokens were cut into steps.
// ---------------------------------------------------------------------------
constexpr int kAttnThreads = 128;

__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(const void* __restrict__ q, int q_dt, const void* __restrict__ k_pages,
                 const void* __restrict__ v_pages, int kv_dt, const int* __restrict__ block_table, int bt_stride,
                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, void* __restrict__ out,
                 int out_dt, int n_heads, int n_kv, int hd, float scale, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                       // hd
    float* p = smem + hd;                   // kAttnThreads
    long long* row = (long long*)(p + kAttnThreads);  // kAttnThreads element offsets of the chunk's rows
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int seq = tok_seq[t];
    const size_t out_base = (size_t)t * n_heads * hd + (size_t)h * hd;
    if (seq < 0) {
        for (int d = tid; d < hd; d += kAttnThreads) st_f(out, out_base + d, out_dt, 0.0f);
        return;
    }
    const int pos = tok_pos[t];
    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int kvh = h / (n_heads / n_kv);
    for (int d = tid; d < hd; d += kAttnThreads) qs[d] = ld_f(q, out_base + d, q_dt);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[8];  // lanes d = tid + 128 * j, hd <= 1024
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;

    for (int k0 = first; k0 <= pos; k0 += kAttnThreads) {
        const int key = k0 + tid;
        float s = -INFINITY;
        long long off = -1;
        if (key <= pos) {
            const int page = block_table[(size_t)seq * bt_stride + key / kPage];
            off = (((long long)page * n_kv + kvh) * kPage + key % kPage) * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], ld_f(k_pages, (size_t)off + d, kv_dt), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float w = key <= pos ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);  // 0 on the first chunk
        l = l * corr + block_sum(w, scratch);
        m = m_new;
        p[tid] = w;
        row[tid] = off;
        __syncthreads();
        const int n_keys = min(kAttnThreads, pos + 1 - k0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = tid + kAttnThreads * j;
            if (d < hd) {
                float a = acc[j] * corr;
                for (int i = 0; i < n_keys; ++i) a = fmaf(p[i], ld_f(v_pages, (size_t)row[i] + d, kv_dt), a);
                acc[j] = a;
            }
        }
        __syncthreads();
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = tid + kAttnThreads * j;
        if (d < hd) st_f(out, out_base + d, out_dt, acc[j] * inv);
    }
}

extern "C" int nncpu_attention(const void* q, int q_dt, const void* k_pages, const void* v_pages, int kv_dt,
                               const int* block_table, int bt_stride, const int* tok_seq, const int* tok_pos,
                               void* out, int out_dt, int n_tok, int n_heads, int n_kv, int hd, float scale,
                               int window, void* stream) {
    NN_CHECK(n_tok >= 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0,
             "attention: %d heads over %d key/value heads", n_heads, n_kv);
    NN_CHECK(hd > 0 && hd <= 1024 && hd % 2 == 0, "attention: head size %d must be even and at most 1024", hd);
    NN_CHECK(window >= 0, "attention: window %d", window);
    if (n_tok == 0) return 0;
    const size_t smem = (hd + kAttnThreads) * sizeof(float) + kAttnThreads * sizeof(long long) + 8;
    dim3 grid(n_tok, n_heads);
    attention_kernel<<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(q, q_dt, k_pages, v_pages, kv_dt,
                                                                         block_table, bt_stride, tok_seq, tok_pos,
                                                                         out, out_dt, n_heads, n_kv, hd, scale,
                                                                         window);
    NN_LAUNCH_OK("attention");
    return 0;
}

// ---------------------------------------------------------------------------
// Gated activation: out[t, i] = silu(gu[t, i]) * gu[t, inter + i].
// ---------------------------------------------------------------------------
__global__ void swiglu_kernel(const void* __restrict__ gu, int in_dt, void* __restrict__ out, int out_dt,
                              long n_tok, int inter) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * inter) return;
    const long t = idx / inter;
    const int i = (int)(idx % inter);
    const float g = ld_f(gu, (size_t)t * 2 * inter + i, in_dt);
    const float u = ld_f(gu, (size_t)t * 2 * inter + inter + i, in_dt);
    st_f(out, (size_t)idx, out_dt, (g * (1.0f / (1.0f + expf(0.0f - g)))) * u);
}

extern "C" int nncpu_swiglu(const void* gu, int in_dt, void* out, int out_dt, int n_tok, int inter, void* stream) {
    NN_CHECK(n_tok >= 0 && inter > 0, "swiglu: %d tokens of %d", n_tok, inter);
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * inter;
    swiglu_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gu, in_dt, out, out_dt, n_tok,
                                                                                      inter);
    NN_LAUNCH_OK("swiglu");
    return 0;
}

// ---------------------------------------------------------------------------
// Gather rows: out[r, :] = x[rows[r], :] (float32), zeros for a negative row.
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int dim) {
    const int r = blockIdx.x, src = rows[r];
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(size_t)r * dim + i] = src < 0 ? 0.0f : x[(size_t)src * dim + i];
}

extern "C" int nncpu_gather_rows(const float* x, const int* rows, float* out, int n_rows, int dim, void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "gather_rows: %d rows of %d", n_rows, dim);
    if (n_rows == 0) return 0;
    gather_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, rows, out, dim);
    NN_LAUNCH_OK("gather_rows");
    return 0;
}

// ---------------------------------------------------------------------------
// Greedy choice: the first largest logit of each row.  NaN never wins.
// ---------------------------------------------------------------------------
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        bv = lane < n_warps ? best_v[lane] : -INFINITY;
        bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// A long row in two steps: blocks (chunk, row) each leave the first largest of their chunk, then one warp per row
// picks among the chunks by the same rule.  One block per row walks 150 000 logits in 33 us whatever the
// number of rows; cut into 32 chunks the two kernels take a few microseconds.
constexpr int kArgmaxChunks = 32;

__global__ void argmax_chunk_kernel(const float* __restrict__ logits, float* __restrict__ part_v,
                                    int* __restrict__ part_i, int vocab) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    const float* row = logits + (size_t)blockIdx.y * vocab;
    const int len = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
    const int begin = blockIdx.x * len, end = min(vocab, begin + len);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        bv = lane < n_warps ? best_v[lane] : -INFINITY;
        bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            part_v[blockIdx.y * kArgmaxChunks + blockIdx.x] = bv;
            part_i[blockIdx.y * kArgmaxChunks + blockIdx.x] = bi;
        }
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                   int* __restrict__ out) {
    static_assert(kArgmaxChunks == 32, "one lane per chunk");
    const int lane = threadIdx.x;
    float bv = part_v[blockIdx.x * kArgmaxChunks + lane];
    int bi = part_i[blockIdx.x * kArgmaxChunks + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// Bytes of scratch that nncpu_argmax wants for rows this long (0: none).
extern "C" long nncpu_argmax_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * kArgmaxChunks * 8 : 0;
}

extern "C" int nncpu_argmax(const float* logits, int* out, int n_rows, int vocab, void* scratch, long scratch_bytes,
                            void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0, "argmax: %d rows of %d", n_rows, vocab);
    if (n_rows == 0) return 0;
    const long need = nncpu_argmax_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need) {
        float* part_v = (float*)scratch;
        int* part_i = (int*)(part_v + (size_t)n_rows * kArgmaxChunks);
        argmax_chunk_kernel<<<dim3(kArgmaxChunks, n_rows), 256, 0, (cudaStream_t)stream>>>(logits, part_v, part_i, vocab);
        NN_LAUNCH_OK("argmax (chunks)");
        argmax_pick_kernel<<<n_rows, 32, 0, (cudaStream_t)stream>>>(part_v, part_i, out);
        NN_LAUNCH_OK("argmax (pick)");
        return 0;
    }
    argmax_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out, vocab);
    NN_LAUNCH_OK("argmax");
    return 0;
}

// ---------------------------------------------------------------------------
// The k best logits of each row in the sampler's ranking: higher logit first,
// then lower id; NaN counts as -inf (crates/nncpu/src/session/sample.rs:69-88,
// 130-152, where a k-element heap makes the same selection).  A radix select
// over the order-preserving integer image of the floats finds the k-th value,
// then everything above it and the lowest ids at it are gathered.  The k
// candidates come out unordered; the host sorts them (k is small).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_order(float v) {
    if (!(v == v)) v = -INFINITY;
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// The selection by radix, for a block of 1024 threads: vals and ids (global or shared memory) receive the k
// candidates of `row` in no particular order.  Works for every row and every k.
__device__ void select_topk_radix(const float* __restrict__ row, int vocab, int k, float* vals, int* ids) {
    __shared__ int hist[256];
    __shared__ uint32_t prefix_s;
    __shared__ int need_s, n_out;
    __shared__ int seg[1024];
    const int tid = threadIdx.x, nt = blockDim.x;
    // radix select, most significant byte first: after 4 rounds `prefix` is the image of the k-th largest value
    uint32_t prefix = 0, mask = 0;
    int need = k;   // how many of the values matching `prefix` so far are still wanted
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += nt) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += nt) {
            const uint32_t u = float_order(row[i]);
            if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int bin = 255, left = need;
            for (; bin > 0; --bin) {
                if (hist[bin] >= left) break;
                left -= hist[bin];
            }
            prefix_s = prefix | ((uint32_t)bin << shift);
            need_s = left;
        }
        __syncthreads();
        prefix = prefix_s;
        need = need_s;
        mask |= 255u << shift;
        __syncthreads();
    }
    // `need` values equal to the k-th value are wanted: the ones with the lowest ids.  Threads own
    // contiguous id ranges so that a scan over the threads counts ties in id order.
    const int per = (vocab + nt - 1) / nt;
    const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
    int ties = 0;
    for (int i = lo; i < hi; ++i) ties += float_order(row[i]) == prefix;
    seg[tid] = ties;
    if (tid == 0) n_out = 0;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < nt; ++i) { const int c = seg[i]; seg[i] = run; run += c; }
    }
    __syncthreads();
    int tie_rank = seg[tid];
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        const uint32_t u = float_order(v);
        bool take = u > prefix;
        if (u == prefix) take = tie_rank++ < need;
        if (take) {
            const int at = atomicAdd(&n_out, 1);
            if (at < k) { vals[at] = (v == v) ? v : -INFINITY; ids[at] = i; }
        }
    }
    __syncthreads();
}

// Ascending bitonic sort of key[0 .. n2) by a block of at least n2 threads; n2 a power of two.
__device__ void sort_keys(unsigned long long* key, int n2) {
    const int tid = threadIdx.x;
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < n2) {
                const int other = tid ^ stride;
                if (other > tid) {
                    const bool up = (tid & size) == 0;
                    const unsigned long long a = key[tid], b = key[other];
                    if ((a > b) == up) { key[tid] = b; key[other] = a; }
                }
            }
            __syncthreads();
        }
    }
}

// (descending logit, ascending id) as one ascending 64-bit key, and back.
__device__ __forceinline__ unsigned long long rank_key(float v, int id) {
    return ((unsigned long long)(~float_order(v)) << 32) | (uint32_t)id;
}
__device__ __forceinline__ float key_value(unsigned long long key) {
    const uint32_t image = ~(uint32_t)(key >> 32);
    return __uint_as_float((image & 0x80000000u) ? (image & 0x7fffffffu) : ~image);
}

// The quick way to the k candidates, which serves the rows a language model produces: the candidates lie within
// 16 of the row's largest logit.  One pass finds the largest, one counts the logits of that range in 1024 bins
// (few logits share a bin there, so the counters do not collide), one gathers everything down to the bin that
// holds the k-th, and a sort of those few puts the k best first.  `key` is scratch for 1024 keys.  Returns
// false, having written nothing, when the range holds fewer than k logits or the gathered ones do not fit:
// then the radix selection does the job.  On success vals and ids are in rank order.
__device__ bool select_topk_near_max(const float* __restrict__ row, int vocab, int k, float* vals, int* ids,
                                     unsigned long long* key) {
    constexpr int kBins = 1024;
    constexpr float kRange = 16.0f, kPerUnit = kBins / kRange;
    __shared__ int fine[kBins];
    __shared__ float red[33];
    __shared__ int cut_bin, n_in, n_got;
    const int tid = threadIdx.x, nt = blockDim.x;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    if (!(mx > -INFINITY) || mx == INFINITY) return false;
    for (int i = tid; i < kBins; i += nt) fine[i] = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += nt) {
        const float d = mx - row[i];
        if (d < kRange) atomicAdd(&fine[(int)(d * kPerUnit)], 1);   // false for NaN
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0, b = 0;
        for (; b < kBins; ++b) {
            run += fine[b];
            if (run >= k) break;
        }
        cut_bin = b;
        n_in = run;
        n_got = 0;
    }
    __syncthreads();
    const int cut = cut_bin, n = n_in;
    if (cut >= kBins || n > 1024) return false;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        const float d = mx - v;
        if (d < kRange && (int)(d * kPerUnit) <= cut) key[atomicAdd(&n_got, 1)] = rank_key(v, i);
    }
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    __syncthreads();
    for (int i = n + tid; i < n2; i += nt) key[i] = ~0ull;
    __syncthreads();
    sort_keys(key, n2);
    if (tid < k) {
        vals[tid] = key_value(key[tid]);
        ids[tid] = (int)(uint32_t)key[tid];
    }
    __syncthreads();
    return true;
}

// The k candidates of `row` in vals and ids; `*sorted` tells whether they came out in rank order.
__device__ void select_topk(const float* __restrict__ row, int vocab, int k, float* vals, int* ids,
                            unsigned long long* key, bool* sorted) {
    *sorted = select_topk_near_max(row, vocab, k, vals, ids, key);
    if (!*sorted) select_topk_radix(row, vocab, k, vals, ids);
}

__global__ void __launch_bounds__(1024)
topk_kernel(const float* __restrict__ logits, float* __restrict__ out_vals, int* __restrict__ out_ids, int vocab, int k) {
    __shared__ unsigned long long key[1024];
    bool sorted;
    select_topk(logits + (size_t)blockIdx.x * vocab, vocab, k, out_vals + (size_t)blockIdx.x * k,
                out_ids + (size_t)blockIdx.x * k, key, &sorted);
}

// ---------------------------------------------------------------------------
// The same candidates for long rows, found by the whole GPU instead of one block per row: a block per
// (chunk, row) for each of the three passes of the quick way (largest logit; counts in 1024 bins within 16 of
// it; gather down to the bin of the k-th), a small kernel between the last two that finds that bin, and the
// chain's kernel then sorts what was gathered.  Per row the scratch holds: the chunks' largest logits, the
// bins, three numbers (the cut bin or -1, how many logits lie down to it, how many were gathered) and 1024 keys.
// ---------------------------------------------------------------------------
constexpr int kPickChunks = 32;
constexpr int kPickBins = 1024;
constexpr float kPickRange = 16.0f, kPickPerUnit = kPickBins / kPickRange;

struct PickScratch {
    float chunk_max[kPickChunks];
    int bins[kPickBins];
    int cut, n_in, n_got, pad;
    unsigned long long key[1024];
};

__device__ __forceinline__ void chunk_span(int vocab, int& begin, int& end) {
    const int len = (vocab + kPickChunks - 1) / kPickChunks;
    begin = blockIdx.x * len;
    end = min(vocab, begin + len);
}

__global__ void __launch_bounds__(256)
pick_max_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    __shared__ float red[33];
    PickScratch& sc = scratch[blockIdx.y];
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    float mx = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    if (threadIdx.x == 0) sc.chunk_max[blockIdx.x] = mx;
    // this block's share of the row's bins and numbers starts at zero
    for (int i = threadIdx.x; i < kPickBins / kPickChunks; i += blockDim.x) sc.bins[blockIdx.x * (kPickBins / kPickChunks) + i] = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) sc.cut = sc.n_in = sc.n_got = 0;
}

__device__ __forceinline__ float row_max_of_chunks(const PickScratch& sc) {
    float mx = -INFINITY;
#pragma unroll 8
    for (int c = 0; c < kPickChunks; ++c) mx = fmaxf(mx, sc.chunk_max[c]);
    return mx;
}

__global__ void __launch_bounds__(256)
pick_count_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    __shared__ int fine[kPickBins];
    PickScratch& sc = scratch[blockIdx.y];
    const float mx = row_max_of_chunks(sc);
    if (!(mx > -INFINITY) || mx == INFINITY) return;
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    for (int i = threadIdx.x; i < kPickBins; i += blockDim.x) fine[i] = 0;
    __syncthreads();
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float d = mx - row[i];
        if (d < kPickRange) atomicAdd(&fine[(int)(d * kPickPerUnit)], 1);   // false for NaN
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPickBins; i += blockDim.x)
        if (fine[i]) atomicAdd(&sc.bins[i], fine[i]);
}

// One block of 1024 threads per row: the bin that holds the k-th logit from the top, by a prefix sum over the bins.
__global__ void __launch_bounds__(kPickBins)
pick_cut_kernel(PickScratch* __restrict__ scratch, int k) {
    __shared__ int warp_total[32];
    PickScratch& sc = scratch[blockIdx.x];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mine = sc.bins[tid];
    int run = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += t;
    }
    if (lane == 31) warp_total[warp] = run;
    __syncthreads();
    if (warp == 0) {
        int t = warp_total[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += v;
        }
        warp_total[lane] = t;
    }
    __syncthreads();
    run += warp > 0 ? warp_total[warp - 1] : 0;     // logits in bins 0 .. tid
    // the first bin whose running count reaches k; none, or too many to gather: -1 (the chain's kernel selects by radix)
    if (run >= k && run - mine < k) {
        sc.cut = run <= 1024 ? tid : -1;
        sc.n_in = run;
    }
    if (tid == kPickBins - 1 && run < k) sc.cut = -1;
}

__global__ void __launch_bounds__(256)
pick_gather_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    PickScratch& sc = scratch[blockIdx.y];
    const int cut = sc.cut;
    const float mx = row_max_of_chunks(sc);
    if (cut < 0 || !(mx > -INFINITY) || mx == INFINITY) return;
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        const float d = mx - v;
        if (d < kPickRange && (int)(d * kPickPerUnit) <= cut) sc.key[atomicAdd(&sc.n_got, 1)] = rank_key(v, i);
    }
}

// ---------------------------------------------------------------------------
// The whole sampling chain of one row on the device, for 0 < top-k <= 1024: the k candidates, their ranking
// (higher logit first, then lower id), top-p and min-p on the distribution at temperature 1, temperature over
// the survivors and the draw in rank order from u[row], uniform in [0, 1)
// (crates/nncpu/src/session/sample.rs:121-201).  After the selection and a bitonic sort one thread walks the
// few candidates with the arithmetic of the reference: 32-bit weights, 64-bit sums.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
sample_chain_kernel(const float* __restrict__ logits, const double* __restrict__ u, int* __restrict__ out, int vocab,
                    int k, float temperature, float top_p, float min_p, const PickScratch* __restrict__ picked) {
    __shared__ float c_val[1024];
    __shared__ int c_id[1024];
    __shared__ unsigned long long key[1024];
    const int tid = threadIdx.x;
    bool sorted;
    if (picked != nullptr && picked[blockIdx.x].cut >= 0) {
        // the candidates were gathered by the kernels before this one: sort them, the k best come first
        const PickScratch& sc = picked[blockIdx.x];
        const int n = sc.n_in;
        int n2 = 1;
        while (n2 < n) n2 <<= 1;
        if (tid < n2) key[tid] = tid < n ? sc.key[tid] : ~0ull;
        __syncthreads();
        sort_keys(key, n2);
        if (tid < k) {
            c_val[tid] = key_value(key[tid]);
            c_id[tid] = (int)(uint32_t)key[tid];
        }
        __syncthreads();
        sorted = true;
    } else {
        select_topk(logits + (size_t)blockIdx.x * vocab, vocab, k, c_val, c_id, key, &sorted);
    }
    if (!sorted) {
        // ascending by (descending logit, ascending id); the padding sorts last
        int n2 = 1;
        while (n2 < k) n2 <<= 1;
        if (tid < n2) key[tid] = tid < k ? rank_key(c_val[tid], c_id[tid]) : ~0ull;
        __syncthreads();
        sort_keys(key, n2);
        if (tid < k) {
            c_val[tid] = key_value(key[tid]);
            c_id[tid] = (int)(uint32_t)key[tid];
        }
        __syncthreads();
    }
    if (tid != 0) return;
    const float top = c_val[0];
    if (!(top > -INFINITY) || top == INFINITY) {   // nothing finite to draw from
        out[blockIdx.x] = c_id[0];
        return;
    }
    // weights at temperature 1
    double total = 0.0;
    for (int i = 0; i < k; ++i) total += (double)expf(c_val[i] - top);
    int keep = k;
    if (top_p > 0.0f && top_p < 1.0f) {
        double cum = 0.0;
        for (int i = 0; i < k; ++i) {
            cum += (double)expf(c_val[i] - top) / total;
            if (cum >= (double)top_p) { keep = i + 1; break; }
        }
    }
    if (min_p > 0.0f) {
        const float floor_ = min_p * 1.0f;   // the best candidate's weight is exp(0) = 1
        int i = 1;
        while (i < keep && expf(c_val[i] - top) >= floor_) ++i;
        keep = i;
    }
    const double inv_t = 1.0 / (double)temperature;
    double sum_t = 0.0;
    for (int i = 0; i < keep; ++i) sum_t += (double)(float)exp((double)(c_val[i] - top) * inv_t);
    double r = u[blockIdx.x] * sum_t;
    int chosen = c_id[keep - 1];
    for (int i = 0; i < keep; ++i) {
        r -= (double)(float)exp((double)(c_val[i] - top) * inv_t);
        if (r <= 0.0) { chosen = c_id[i]; break; }
    }
    out[blockIdx.x] = chosen;
}

// Bytes of scratch with which nncpu_sample_chain finds the candidates of long rows by the whole GPU (0: rows
// are short, one block per row does it all).
extern "C" long nncpu_sample_chain_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * (long)sizeof(PickScratch) : 0;
}

extern "C" int nncpu_sample_chain(const float* logits, const double* u, int* out, int n_rows, int vocab, int top_k,
                                  float temperature, float top_p, float min_p, void* scratch, long scratch_bytes,
                                  void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(n_rows >= 0 && vocab > 0, "sample_chain: %d rows of %d", n_rows, vocab);
    NN_CHECK(top_k > 0 && top_k <= 1024 && top_k <= vocab, "sample_chain: top-k %d is outside 1..min(1024, %d)", top_k, vocab);
    NN_CHECK(temperature > 0.0f && temperature < INFINITY, "sample_chain: temperature %g", (double)temperature);
    NN_CHECK(top_p >= 0.0f && top_p <= 1.0f && min_p >= 0.0f && min_p <= 1.0f, "sample_chain: top-p %g, min-p %g",
             (double)top_p, (double)min_p);
    if (n_rows == 0) return 0;
    PickScratch* picked = nullptr;
    const long need = nncpu_sample_chain_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need && ((uintptr_t)scratch % 8) == 0) {
        picked = (PickScratch*)scratch;
        const dim3 grid(kPickChunks, n_rows);
        pick_max_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (largest)");
        pick_count_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (count)");
        pick_cut_kernel<<<n_rows, kPickBins, 0, stream>>>(picked, top_k);
        NN_LAUNCH_OK("sample_chain (cut)");
        pick_gather_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (gather)");
    }
    sample_chain_kernel<<<n_rows, 1024, 0, stream>>>(logits, u, out, vocab, top_k, temperature, top_p, min_p, picked);
    NN_LAUNCH_OK("sample_chain");
    return 0;
}

// Per row: sum over the vocabulary of exp(logit - largest logit), NaN as -inf: the denominator of the
// distribution at temperature 1, which top-p and min-p are measured on.
__global__ void __launch_bounds__(1024)
row_exp_sum_kernel(const float* __restrict__ logits, double* __restrict__ out_sum, int vocab) {
    __shared__ float red_f[32];
    __shared__ double red_d[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v) m = fmaxf(m, v);
    }
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red_f[warp] = m;
    __syncthreads();
    m = red_f[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red_f[w]);
    double s = 0.0;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v && v != -INFINITY) s += (double)expf(v - m);
    }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red_d[warp] = s;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red_d[w];
        out_sum[blockIdx.x] = t;
    }
}

extern "C" int nncpu_row_exp_sum(const float* logits, double* out_sum, int n_rows, int vocab, void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0, "row_exp_sum: %d rows of %d", n_rows, vocab);
    if (n_rows == 0) return 0;
    row_exp_sum_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out_sum, vocab);
    NN_LAUNCH_OK("row_exp_sum");
    return 0;
}

extern "C" int nncpu_topk(const float* logits, float* out_vals, int* out_ids, int n_rows, int vocab, int k, void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0 && k > 0 && k <= vocab, "topk: %d rows of %d, k %d", n_rows, vocab, k);
    if (n_rows == 0) return 0;
    topk_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out_vals, out_ids, vocab, k);
    NN_LAUNCH_OK("topk");
    return 0;
}

// ---------------------------------------------------------------------------
// Temperature draw over the whole vocabulary, in token-id order:
// p_i = exp((l_i - max) / T) in double, r = u * sum(p), the first i whose
// running sum reaches r.  NaN counts as -inf.  `u[row]` is uniform in [0, 1).
// ---------------------------------------------------------------------------
__global__ void sample_kernel(const float* __restrict__ logits, const double* __restrict__ u,
                              int* __restrict__ out, int vocab, float inv_temp) {
    __shared__ float scratch[33];
    __shared__ double part[1024];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, nt = blockDim.x;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, scratch);
    if (!(mx > -INFINITY) || mx == INFINITY) {  // nothing finite to draw from: the first largest
        if (tid == 0) {
            int best = 0;
            for (int i = 1; i < vocab; ++i) if (row[i] > row[best] || (row[best] != row[best] && row[i] == row[i])) best = i;
            out[blockIdx.x] = best;
        }
        return;
    }
    // thread `tid` owns the contiguous ids [lo, hi)
    const int per = (vocab + nt - 1) / nt;
    const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
    }
    part[tid] = s;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int i = 0; i < nt; ++i) total += part[i];
        double r = u[blockIdx.x] * total;
        int owner = nt - 1;
        for (int i = 0; i < nt; ++i) {
            if (r - part[i] <= 0.0 && part[i] > 0.0) { owner = i; break; }
            r -= part[i];
        }
        // walk the owner's ids; the last id with weight is the fallback
        const int olo = min(vocab, owner * per), ohi = min(vocab, olo + per);
        int pick = -1, last = -1;
        for (int i = olo; i < ohi; ++i) {
            const float v = row[i];
            if (!(v == v)) continue;
            const double w = exp((double)(v - mx) * (double)inv_temp);
            if (w > 0.0) last = i;
            r -= w;
            if (r <= 0.0 && w > 0.0) { pick = i; break; }
        }
        if (pick < 0) pick = last;
        if (pick < 0) {  // rounding pushed r past the end: the last id with weight anywhere
            for (int i = vocab - 1; i >= 0; --i) {
                const float v = row[i];
                if (v == v && exp((double)(v - mx) * (double)inv_temp) > 0.0) { pick = i; break; }
            }
        }
        out[blockIdx.x] = pick < 0 ? 0 : pick;
    }
}

// The same draw for long rows in three kernels: the chunks' largest logits (pick_max_kernel), the chunks' sums
// of weights, and a block per row that finds the chunk in which the running sum reaches r and walks that chunk
// alone.  Per row the scratch is a PickScratch; the chunk sums lie where its keys would.
__global__ void __launch_bounds__(256)
sample_chunk_sum_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab, float inv_temp) {
    __shared__ double red[8];
    PickScratch& sc = scratch[blockIdx.y];
    const float mx = row_max_of_chunks(sc);
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    double s = 0.0;
    if (mx > -INFINITY && mx != INFINITY) {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
        }
    }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        reinterpret_cast<double*>(sc.key)[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256)
sample_chunk_draw_kernel(const float* __restrict__ logits, const double* __restrict__ u, int* __restrict__ out,
                         const PickScratch* __restrict__ scratch, int vocab, float inv_temp) {
    __shared__ double part[256];
    const PickScratch& sc = scratch[blockIdx.x];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, nt = blockDim.x;
    const float mx = row_max_of_chunks(sc);
    if (!(mx > -INFINITY) || mx == INFINITY) {  // nothing finite to draw from: the first largest
        if (tid == 0) {
            int best = 0;
            for (int i = 1; i < vocab; ++i) if (row[i] > row[best] || (row[best] != row[best] && row[i] == row[i])) best = i;
            out[blockIdx.x] = best;
        }
        return;
    }
    // the chunk in which the running sum, in id order, reaches r; the last chunk with weight if rounding ran past the end
    const double* chunk_sum = reinterpret_cast<const double*>(sc.key);
    double total = 0.0;
    for (int c = 0; c < kPickChunks; ++c) total += chunk_sum[c];
    double r = u[blockIdx.x] * total;
    int chunk = -1, last_chunk = -1;
    for (int c = 0; c < kPickChunks; ++c) {
        if (chunk_sum[c] > 0.0) last_chunk = c;
        if (r - chunk_sum[c] <= 0.0 && chunk_sum[c] > 0.0) { chunk = c; break; }
        r -= chunk_sum[c];
    }
    if (chunk < 0) {      // past the end: the last id with weight
        chunk = last_chunk;
        r = INFINITY;
    }
    if (chunk < 0) {      // no weight anywhere (cannot be: the largest logit has weight 1)
        if (tid == 0) out[blockIdx.x] = 0;
        return;
    }
    const int len = (vocab + kPickChunks - 1) / kPickChunks;
    const int begin = chunk * len, end = min(vocab, begin + len);
    // thread `tid` owns the contiguous ids [lo, hi) of the chunk
    const int per = (end - begin + nt - 1) / nt;
    const int lo = min(end, begin + tid * per), hi = min(end, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
    }
    part[tid] = s;
    __syncthreads();
    if (tid != 0) return;
    int owner = -1, last_owner = -1;
    for (int i = 0; i < nt; ++i) {
        if (part[i] > 0.0) last_owner = i;
        if (r - part[i] <= 0.0 && part[i] > 0.0) { owner = i; break; }
        r -= part[i];
    }
    if (owner < 0) {
        owner = last_owner;
        r = INFINITY;
    }
    int pick = -1, last = -1;
    if (owner >= 0) {
        const int olo = min(end, begin + owner * per), ohi = min(end, olo + per);
        for (int i = olo; i < ohi; ++i) {
            const float v = row[i];
            if (!(v == v)) continue;
            const double w = exp((double)(v - mx) * (double)inv_temp);
            if (w > 0.0) last = i;
            r -= w;
            if (r <= 0.0 && w > 0.0) { pick = i; break; }
        }
    }
    if (pick < 0) pick = last;
    out[blockIdx.x] = pick < 0 ? 0 : pick;
}

extern "C" long nncpu_sample_temperature_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * (long)sizeof(PickScratch) : 0;
}

extern "C" int nncpu_sample_temperature(const float* logits, const double* u, int* out, int n_rows, int vocab,
                                        float temperature, void* scratch, long scratch_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(n_rows >= 0 && vocab > 0, "sample: %d rows of %d", n_rows, vocab);
    NN_CHECK(temperature > 0.0f && isfinite(temperature), "sample: temperature %g must be positive", temperature);
    if (n_rows == 0) return 0;
    const long need = nncpu_sample_temperature_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need && ((uintptr_t)scratch % 8) == 0) {
        PickScratch* sc = (PickScratch*)scratch;
        const dim3 grid(kPickChunks, n_rows);
        pick_max_kernel<<<grid, 256, 0, stream>>>(logits, sc, vocab);
        NN_LAUNCH_OK("sample (largest)");
        sample_chunk_sum_kernel<<<grid, 256, 0, stream>>>(logits, sc, vocab, 1.0f / temperature);
        NN_LAUNCH_OK("sample (sums)");
        sample_chunk_draw_kernel<<<n_rows, 256, 0, stream>>>(logits, u, out, sc, vocab, 1.0f / temperature);
        NN_LAUNCH_OK("sample (draw)");
        return 0;
    }
    sample_kernel<<<n_rows, 1024, 0, stream>>>(logits, u, out, vocab, 1.0f / temperature);
    NN_LAUNCH_OK("sample");
    return 0;
}
