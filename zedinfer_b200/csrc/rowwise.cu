// Row-wise kernels beside those of elementwise.cu: embedding with a learned position table, the logit cap,
// two feed-forward activations (squared ReLU; a clamped, sigmoid-gated product), and an RMSNorm whose output
// rows go straight into the pages of a paged cache (the latent of a latent-attention layer).
// All arithmetic is float32; storage types are float32 or bfloat16 per tensor.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(rowwise)

// ---------------------------------------------------------------------------------------
// Embedding with learned absolute positions: out[n, :] = table[ids[n], :] + pos_table[pos[n], :]
// ---------------------------------------------------------------------------------------
template <typename TT, typename TO>
__global__ void embedding_pos_kernel(const TT* __restrict__ table, const TT* __restrict__ pos_table,
                                     const int* __restrict__ ids, const int* __restrict__ pos, TO* __restrict__ out,
                                     int hidden, int vocab, int max_pos) {
    const int n = blockIdx.x;
    int id = ids[n], p = pos[n];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);       // the host refuses ids and positions outside the tables
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    const TT* src = table + (size_t)id * hidden;
    const TT* ps = pos_table + (size_t)p * hidden;
    TO* dst = out + (size_t)n * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = from_f32<TO>(to_f32<TT>(src[j]) + to_f32<TT>(ps[j]));
}

ZI_EXPORT int zi_embedding_pos(const void* table, const void* pos_table, int table_dtype, const int* ids, const int* pos,
                               void* out, int out_dtype, int n_tokens, int hidden, int vocab, int max_pos,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || max_pos <= 0)
        return zi_fail("embedding: hidden=%d vocab=%d positions=%d must be positive", hidden, vocab, max_pos);
    const int threads = hidden >= 1024 ? 256 : 128;
    ZI_DISPATCH(table_dtype, TT, ZI_DISPATCH(out_dtype, TO, {
        embedding_pos_kernel<TT, TO><<<n_tokens, threads, 0, stream>>>((const TT*)table, (const TT*)pos_table, ids, pos,
                                                                      (TO*)out, hidden, vocab, max_pos);
    }););
    return zi_check_launch("embedding_pos");
}

// ---------------------------------------------------------------------------------------
// Logit cap, in place on float32: x = cap * tanh(x / cap)
// ---------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

ZI_EXPORT int zi_softcap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.0f)) return zi_fail("softcap: cap=%g must be positive", (double)cap);
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    softcap_kernel<<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>(x, (size_t)total, cap);
    return zi_check_launch("softcap");
}

// ---------------------------------------------------------------------------------------
// Squared ReLU: out = max(x, 0)^2
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32<T>(x[i]), 0.0f);
        out[i] = from_f32<T>(v * v);
    }
}
template <typename T>
__global__ void relu2_vec8_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        float v[8];
        load8(x + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[e] = fmaxf(v[e], 0.0f); v[e] = v[e] * v[e]; }
        store8(out + i * 8, v);
    }
}

ZI_EXPORT int zi_relu2(const void* x, void* out, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    if (total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 31) == 0) {
        const long long want = (total / 8 + threads - 1) / threads;
        ZI_DISPATCH(dtype, T, { relu2_vec8_kernel<T><<<(int)(want > 148 * 32 ? 148 * 32 : want), threads, 0, stream>>>((const T*)x, (T*)out, (size_t)(total / 8)); });
        return zi_check_launch("relu2");
    }
    const long long want = (total + threads - 1) / threads;
    ZI_DISPATCH(dtype, T, { relu2_kernel<T><<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>((const T*)x, (T*)out, (size_t)total); });
    return zi_check_launch("relu2");
}

// ---------------------------------------------------------------------------------------
// Clamped gated product.  x [rows, 2 * inter]: gate = x[n, j], up = x[n, inter + j];
//   g = min(gate, limit);  u = clamp(up, -limit, limit);  out[n, j] = g * sigmoid(slope * g) * (u + up_offset)
// limit <= 0: no clamping.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float clamped_gate(float g, float u, float limit, float slope, float up_offset) {
    if (limit > 0.0f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return (g / (1.0f + expf(-slope * g))) * (u + up_offset);
}

template <typename T>
__global__ void gated_clamp_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, size_t total,
                                       float limit, float slope, float up_offset) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter, j = i - n * inter;
        out[i] = from_f32<T>(clamped_gate(to_f32<T>(x[n * 2 * inter + j]), to_f32<T>(x[n * 2 * inter + inter + j]),
                                          limit, slope, up_offset));
    }
}
template <typename T>
__global__ void gated_clamp_mul_vec8_kernel(const T* __restrict__ x, T* __restrict__ out, int inter8, size_t total8,
                                            float limit, float slope, float up_offset) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter8, j = (i - n * inter8) * 8;
        const size_t inter = (size_t)inter8 * 8;
        float g[8], u[8], r[8];
        load8(x + n * 2 * inter + j, g);
        load8(x + n * 2 * inter + inter + j, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = clamped_gate(g[e], u[e], limit, slope, up_offset);
        store8(out + n * inter + j, r);
    }
}

ZI_EXPORT int zi_gated_clamp_mul(const void* gate_up, void* out, int dtype, int rows, int inter, float limit, float slope,
                                 float up_offset, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) return zi_fail("gated_clamp_mul: width %d must be positive", inter);
    const size_t total = (size_t)rows * inter;
    const int threads = 256;
    if (inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 31) == 0) {
        const size_t total8 = total / 8;
        const size_t want = (total8 + threads - 1) / threads;
        ZI_DISPATCH(dtype, T, {
            gated_clamp_mul_vec8_kernel<T><<<(int)(want > 148 * 32 ? 148 * 32 : want), threads, 0, stream>>>(
                (const T*)gate_up, (T*)out, inter / 8, total8, limit, slope, up_offset);
        });
        return zi_check_launch("gated_clamp_mul");
    }
    const size_t want = (total + threads - 1) / threads;
    ZI_DISPATCH(dtype, T, {
        gated_clamp_mul_kernel<T><<<(int)(want > 148 * 16 ? 148 * 16 : want), threads, 0, stream>>>(
            (const T*)gate_up, (T*)out, inter, total, limit, slope, up_offset);
    });
    return zi_check_launch("gated_clamp_mul");
}

// ---------------------------------------------------------------------------------------
// RMSNorm of `width` columns of each row of x, written into the pages of a paged cache with one
// plane and one head per token (a latent):  y = (w * x) * rstd,  rstd = 1/sqrt(mean(x^2) + eps).
//   x      [n_tokens, row_stride]; the first `width` columns of a row are normed
//   cache  one call's slice of the pool: row (page, off) is at cache + page*page_stride + off*width
//   tables [n_segments, max_blocks] page ids; tok_seg[n] = segment of token n; pos[n] = its position
// One warp per token; the sum's order depends on the width alone.
// ---------------------------------------------------------------------------------------
#define NA_WARPS 4
template <typename TX, typename TW, typename TC>
__global__ void __launch_bounds__(NA_WARPS * 32)
rmsnorm_append_kernel(const TX* __restrict__ x, long long row_stride, const TW* __restrict__ w, float eps,
                      TC* __restrict__ cache, const int* __restrict__ tables, const int* __restrict__ tok_seg,
                      const int* __restrict__ pos, int n_tokens, int width, int page_size, int max_blocks,
                      long long page_stride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * NA_WARPS + warp;
    if (n >= n_tokens) return;
    const TX* xr = x + (size_t)n * row_stride;
    float ss = 0.0f;
    for (int j = lane; j < width; j += 32) {
        const float v = to_f32<TX>(xr[j]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
    const int p = pos[n];
    const int seg = tok_seg ? tok_seg[n] : n;
    const int page = tables[(size_t)seg * max_blocks + p / page_size];
    TC* dst = cache + (long long)page * page_stride + (long long)(p % page_size) * width;
    for (int j = lane; j < width; j += 32) dst[j] = from_f32<TC>((to_f32<TW>(w[j]) * to_f32<TX>(xr[j])) * rstd);
}

ZI_EXPORT int zi_rmsnorm_append(const void* x, int x_dtype, long long row_stride, const void* w, int w_dtype, float eps,
                                void* cache, int cache_dtype, const int* tables, const int* tok_seg, const int* pos,
                                int n_tokens, int width, int page_size, int max_blocks, long long page_stride,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (width <= 0 || row_stride < width) return zi_fail("rmsnorm_append: width=%d row_stride=%lld", width, row_stride);
    if (page_size <= 0 || max_blocks <= 0) return zi_fail("rmsnorm_append: page_size=%d max_blocks=%d", page_size, max_blocks);
    const int blocks = (n_tokens + NA_WARPS - 1) / NA_WARPS;
    ZI_DISPATCH(x_dtype, TX, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(cache_dtype, TC, {
        rmsnorm_append_kernel<TX, TW, TC><<<blocks, NA_WARPS * 32, 0, stream>>>(
            (const TX*)x, row_stride, (const TW*)w, eps, (TC*)cache, tables, tok_seg, pos, n_tokens, width, page_size,
            max_blocks, page_stride);
    });););
    return zi_check_launch("rmsnorm_append");
}
