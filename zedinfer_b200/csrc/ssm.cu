// Kernels of a selective state-space mixer (Mamba-2 form) over the tokens of one step:
//
//   zi_segment_bounds       first and past-the-last token of every segment, from the token -> segment map
//   zi_causal_conv_silu     short causal convolution per channel with bias and SiLU; what lies before a segment's
//                           portion comes from the request's state slot, what lies before position 0 is zero
//   zi_conv_state_update    the last taps - 1 inputs of every segment go into its state slot
//   zi_ssm_scan             S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t, token by token,
//                           the state read from and written back to the request's slot
//   zi_gated_group_rmsnorm  out = unit_rms_per_group(y * silu(z)) * w
//
// Everything that enters the recurrence is float32: step sizes (softplus, no clamp), decays, the state, the sums.
// Every sum has one order that depends on the sizes alone, so a token's result does not depend on how its request
// was cut into steps or on what else is in the batch.
//
// A request's state slot (float32) holds the recurrent state, laid out [heads, vdim, state] (a column's entries are
// consecutive), and behind it the convolution's ring [taps - 1, channels]: the input at position q is in row
// q mod (taps - 1).  Slot -1 (a row of padding): the state is zero and nothing is written.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(ssm)

// ---------------------------------------------------------------------------------------
__global__ void segment_bounds_kernel(const int* __restrict__ tok_seg, int n_tokens, int* __restrict__ bounds) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= n_tokens) return;
    const int s = tok_seg[n];
    if (n == 0 || tok_seg[n - 1] != s) bounds[2 * s] = n;
    if (n == n_tokens - 1 || tok_seg[n + 1] != s) bounds[2 * s + 1] = n + 1;
}

ZI_EXPORT int zi_segment_bounds(const int* tok_seg, int n_tokens, int n_segments, int* bounds, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segments <= 0) return 0;
    cudaMemsetAsync(bounds, 0, (size_t)n_segments * 2 * sizeof(int), stream);
    segment_bounds_kernel<<<(n_tokens + 255) / 256, 256, 0, stream>>>(tok_seg, n_tokens, bounds);
    return zi_check_launch("segment_bounds");
}

// ---------------------------------------------------------------------------------------
// out[n, c] = silu(bias[c] + sum_j w[c, j] * u(pos[n] - (taps - 1) + j)), j rising; u from this step's rows where the
// position lies in the segment's portion, else from the slot's ring, zero before position 0.
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void causal_conv_silu_kernel(const T* __restrict__ u, long long ldu, const TW* __restrict__ w,
                                        const TW* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                                        const int* __restrict__ slots, const int* __restrict__ tok_seg,
                                        const int* __restrict__ pos, T* __restrict__ out, int n_tokens, int channels, int taps) {
    const int n = blockIdx.y;
    const int seg = tok_seg ? tok_seg[n] : n;
    const int p = pos[n];
    const int slot = slots[seg];
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        float acc = bias ? to_f32<TW>(bias[c]) : 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;
            const int q = p - back;
            if (q < 0) continue;
            float v;
            const bool here = back == 0 || (n - back >= 0 && (tok_seg ? tok_seg[n - back] == seg : false));
            if (here) v = to_f32<T>(u[(size_t)(n - back) * ldu + c]);
            else v = slot >= 0 ? state[(size_t)slot * slot_stride + (size_t)(q % (taps - 1)) * channels + c] : 0.0f;
            acc = fmaf(to_f32<TW>(w[(size_t)c * taps + j]), v, acc);
        }
        out[(size_t)n * channels + c] = from_f32<T>(acc / (1.0f + expf(-acc)));
    }
}

ZI_EXPORT int zi_causal_conv_silu(const void* u, int dtype, long long ldu, const void* w, const void* bias, int w_dtype,
                                  const float* state, long long slot_stride, const int* slots, const int* tok_seg,
                                  const int* pos, void* out, int n_tokens, int channels, int taps, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps <= 0) return zi_fail("causal_conv: taps=%d must be positive", taps);
    if (n_tokens > 65535 * 32) return zi_fail("causal_conv: too many tokens for one launch");
    dim3 grid((channels + 255) / 256, n_tokens);
    if (grid.y > 65535) return zi_fail("causal_conv: %d tokens are too many for one launch", n_tokens);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        causal_conv_silu_kernel<T, TW><<<grid, 256, 0, stream>>>((const T*)u, ldu, (const TW*)w, (const TW*)bias, state, slot_stride,
                                                                 slots, tok_seg, pos, (T*)out, n_tokens, channels, taps);
    }););
    return zi_check_launch("causal_conv_silu");
}

// One thread per (segment, channel): the last min(taps - 1, portion) inputs go into the ring.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ u, long long ldu, float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ slots, const int* __restrict__ bounds,
                                         const int* __restrict__ pos, int channels, int taps) {
    const int seg = blockIdx.y;
    const int slot = slots[seg];
    if (slot < 0) return;
    const int first = bounds ? bounds[2 * seg] : seg, end = bounds ? bounds[2 * seg + 1] : seg + 1;
    const int keep = end - first < taps - 1 ? end - first : taps - 1;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x)
        for (int d = 0; d < keep; ++d) {
            const int n = end - 1 - d;
            state[(size_t)slot * slot_stride + (size_t)(pos[n] % (taps - 1)) * channels + c] = to_f32<T>(u[(size_t)n * ldu + c]);
        }
}

ZI_EXPORT int zi_conv_state_update(const void* u, int dtype, long long ldu, float* state, long long slot_stride, const int* slots,
                                   const int* bounds, const int* pos, int n_segments, int channels, int taps, cudaStream_t stream) {
    if (n_segments <= 0 || channels <= 0 || taps <= 1) return 0;
    dim3 grid((channels + 255) / 256, n_segments);
    if (grid.y > 65535) return zi_fail("conv_state_update: %d segments are too many for one launch", n_segments);
    ZI_DISPATCH(dtype, T, {
        conv_state_update_kernel<T><<<grid, 256, 0, stream>>>((const T*)u, ldu, state, slot_stride, slots, bounds, pos, channels, taps);
    });
    return zi_check_launch("conv_state_update");
}

// ---------------------------------------------------------------------------------------
// The scan.  A block takes (segment, head, a tile of the head's columns p) and walks the segment's tokens in order.
// A column's state entries are dealt to L lanes of a warp (L a power of two, R = ceil(N / L) <= 16 entries each, lane l
// holding n = l R .. l R + R - 1), so a warp holds 32 / L columns.  Tokens come in chunks: B, C, x, the step sizes and
// the decays of a chunk are put into shared memory by the whole block, then every thread walks the chunk.
// ---------------------------------------------------------------------------------------
#define SCAN_R 16
#define SCAN_CHUNK 32

__device__ __forceinline__ float softplus_f32(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

template <typename T, typename TP>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ dt_in, long long ld_dt,
                const TP* __restrict__ dt_bias, const TP* __restrict__ a_log, const TP* __restrict__ d_skip,
                float* __restrict__ state, long long slot_stride, const int* __restrict__ slots,
                const int* __restrict__ bounds, float* __restrict__ y, int heads, int vdim, int N, int groups,
                int L, int R, int chunk) {
    extern __shared__ float sm[];
    const int seg = blockIdx.x, h = blockIdx.y;
    const int warps = blockDim.x >> 5, pt = 32 / L, pc = warps * pt;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nl = lane % L, col = warp * pt + lane / L;
    const int p = blockIdx.z * pc + col;
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const int first = bounds ? bounds[2 * seg] : seg, end = bounds ? bounds[2 * seg + 1] : seg + 1;
    const int slot = slots[seg];
    float* Bs = sm;                         // [chunk][N]
    float* Cs = Bs + (size_t)chunk * N;     // [chunk][N]
    float* xs = Cs + (size_t)chunk * N;     // [chunk][pc]
    float* dts = xs + (size_t)chunk * pc;   // [chunk]
    float* decs = dts + chunk;              // [chunk]
    const float a_rate = expf(to_f32<TP>(a_log[h])), bias = to_f32<TP>(dt_bias[h]), skip = to_f32<TP>(d_skip[h]);
    const bool live = p < vdim;
    float S[SCAN_R];
    float* srow = (slot >= 0 && live) ? state + (size_t)slot * slot_stride + ((size_t)h * vdim + p) * N + (size_t)nl * R : nullptr;
#pragma unroll
    for (int r = 0; r < SCAN_R; ++r) S[r] = (srow && r < R && nl * R + r < N) ? srow[r] : 0.0f;
    for (int t0 = first; t0 < end; t0 += chunk) {
        const int cnt = end - t0 < chunk ? end - t0 : chunk;
        __syncthreads();
        for (int i = threadIdx.x; i < cnt * N; i += blockDim.x) {
            const int t = i / N, n = i - t * N;
            const T* row = xbc + (size_t)(t0 + t) * ldx + inner + (size_t)g * N + n;
            Bs[i] = to_f32<T>(row[0]);
            Cs[i] = to_f32<T>(row[(size_t)groups * N]);
        }
        for (int i = threadIdx.x; i < cnt * pc; i += blockDim.x) {
            const int t = i / pc, c = i - t * pc;
            const int pp = blockIdx.z * pc + c;
            xs[i] = pp < vdim ? to_f32<T>(xbc[(size_t)(t0 + t) * ldx + (size_t)h * vdim + pp]) : 0.0f;
        }
        for (int t = threadIdx.x; t < cnt; t += blockDim.x) {
            const float dt = softplus_f32(to_f32<T>(dt_in[(size_t)(t0 + t) * ld_dt + h]) + bias);
            dts[t] = dt;
            decs[t] = expf(-a_rate * dt);
        }
        __syncthreads();
        for (int t = 0; t < cnt; ++t) {
            const float a = decs[t], xv = xs[t * pc + col], dx = dts[t] * xv;
            const float* bt = Bs + (size_t)t * N + nl * R;
            const float* ct = Cs + (size_t)t * N + nl * R;
            float acc = 0.0f;
#pragma unroll
            for (int r = 0; r < SCAN_R; ++r) {
                if (r < R && nl * R + r < N) {
                    S[r] = fmaf(dx, bt[r], a * S[r]);
                    acc = fmaf(S[r], ct[r], acc);
                }
            }
            for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (nl == 0 && live) y[(size_t)(t0 + t) * inner + (size_t)h * vdim + p] = fmaf(skip, xv, acc);
        }
    }
    if (srow) {
#pragma unroll
        for (int r = 0; r < SCAN_R; ++r)
            if (r < R && nl * R + r < N) srow[r] = S[r];
    }
}

ZI_EXPORT int zi_ssm_scan(const void* xbc, int dtype, long long ldx, const void* dt_in, long long ld_dt, const void* dt_bias,
                          const void* a_log, const void* d_skip, int p_dtype, float* state, long long slot_stride,
                          const int* slots, const int* bounds, float* y, int n_segments, int heads, int vdim, int N,
                          int groups, cudaStream_t stream) {
    if (n_segments <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || N <= 0 || groups <= 0 || heads % groups)
        return zi_fail("ssm_scan: heads=%d vdim=%d state=%d groups=%d", heads, vdim, N, groups);
    int L = 1;
    while ((N + L - 1) / L > SCAN_R && L < 32) L *= 2;
    const int R = (N + L - 1) / L;
    if (R > SCAN_R) return zi_fail("ssm_scan: state=%d is more than %d", N, 32 * SCAN_R);
    const int pt = 32 / L;
    int warps = (vdim + pt - 1) / pt;
    if (warps > 8) warps = 8;
    const int pc = warps * pt;
    const int ptiles = (vdim + pc - 1) / pc;
    int chunk = SCAN_CHUNK;
    while (chunk > 1 && ((size_t)chunk * (2 * N + pc + 2)) * sizeof(float) > 40 * 1024) chunk /= 2;
    const size_t smem = ((size_t)chunk * (2 * N + pc + 2)) * sizeof(float);
    if (smem > 48 * 1024) return zi_fail("ssm_scan: state=%d needs %zu bytes of shared memory", N, smem);
    if (heads > 65535 || ptiles > 65535) return zi_fail("ssm_scan: too many heads or columns for one launch");
    dim3 grid(n_segments, heads, ptiles);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(p_dtype, TP, {
        ssm_scan_kernel<T, TP><<<grid, warps * 32, smem, stream>>>((const T*)xbc, ldx, (const T*)dt_in, ld_dt, (const TP*)dt_bias,
                                                                   (const TP*)a_log, (const TP*)d_skip, state, slot_stride, slots,
                                                                   bounds, y, heads, vdim, N, groups, L, R, chunk);
    }););
    return zi_check_launch("ssm_scan");
}

// ---------------------------------------------------------------------------------------
// out[n, :] = unit_rms_per_group(y[n, :] * silu(z[n, :])) * w, float32 inside; a block per (token, group).
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long ldz,
                                           const TW* __restrict__ w, T* __restrict__ out, int inner, int group_size, float eps) {
    __shared__ float scratch[32];
    const int n = blockIdx.x, g = blockIdx.y;
    const float* yr = y + (size_t)n * inner + (size_t)g * group_size;
    const T* zr = z + (size_t)n * ldz + (size_t)g * group_size;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < group_size; j += blockDim.x) {
        const float zv = to_f32<T>(zr[j]);
        const float v = yr[j] * (zv / (1.0f + expf(-zv)));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)group_size + eps);
    for (int j = threadIdx.x; j < group_size; j += blockDim.x) {
        const float zv = to_f32<T>(zr[j]);
        const float v = yr[j] * (zv / (1.0f + expf(-zv)));
        out[(size_t)n * inner + (size_t)g * group_size + j] = from_f32<T>(v * inv * to_f32<TW>(w[(size_t)g * group_size + j]));
    }
}

ZI_EXPORT int zi_gated_group_rmsnorm(const float* y, const void* z, int dtype, long long ldz, const void* w, int w_dtype, void* out,
                                     int n_tokens, int inner, int n_groups, float eps, cudaStream_t stream) {
    if (n_tokens <= 0 || inner <= 0) return 0;
    if (n_groups <= 0 || inner % n_groups) return zi_fail("gated_group_rmsnorm: %d groups do not divide %d", n_groups, inner);
    const int gs = inner / n_groups;
    if (n_groups > 65535) return zi_fail("gated_group_rmsnorm: too many groups");
    const int threads = gs >= 1024 ? 256 : 128;
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        gated_group_rmsnorm_kernel<T, TW><<<dim3(n_tokens, n_groups), threads, 0, stream>>>(y, (const T*)z, ldz, (const TW*)w, (T*)out,
                                                                                           inner, gs, eps);
    }););
    return zi_check_launch("gated_group_rmsnorm");
}
