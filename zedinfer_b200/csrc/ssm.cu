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
// update_state (a step of single tokens only, tok_seg null): the kernel also puts every token's input into its ring, which
// zi_conv_state_update does otherwise.
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void causal_conv_silu_kernel(const T* __restrict__ u, long long ldu, const TW* __restrict__ w,
                                        const TW* __restrict__ bias, const float* state, long long slot_stride,
                                        const int* __restrict__ slots, const int* __restrict__ tok_seg,
                                        const int* __restrict__ pos, T* __restrict__ out, int n_tokens, int channels, int taps,
                                        float* ring   /* the same memory as `state` when given: no restrict on either */) {
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
        // a step of single tokens: this thread alone read its channel's ring, so it may put the token's input there itself
        if (ring && slot >= 0 && taps > 1)
            ring[(size_t)slot * slot_stride + (size_t)(p % (taps - 1)) * channels + c] = to_f32<T>(u[(size_t)n * ldu + c]);
    }
}

// The same, eight neighbouring channels per thread with 16- or 32-byte accesses (channels % 8 == 0, aligned rows); the same
// sums in the same order.
template <typename T, typename TW, int TAPS>
__global__ void causal_conv_silu_vec8_kernel(const T* __restrict__ u, long long ldu, const TW* __restrict__ w,
                                             const TW* __restrict__ bias, const float* state, long long slot_stride,
                                             const int* __restrict__ slots, const int* __restrict__ tok_seg,
                                             const int* __restrict__ pos, T* __restrict__ out, int n_tokens, int channels, int taps,
                                             float* ring   /* the same memory as `state` when given: no restrict on either */) {
    const int n = blockIdx.y;
    const int seg = tok_seg ? tok_seg[n] : n;
    const int p = pos[n];
    const int slot = slots[seg];
    if (TAPS > 0) taps = TAPS;
    for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8; c < channels; c += gridDim.x * blockDim.x * 8) {
        float acc[8];
        // the eight channels' weights are 8 * taps consecutive values: whole vectors where the number of taps is known
        float wv[TAPS > 0 ? TAPS : 1][8];
        if (TAPS > 0) {
#pragma unroll
            for (int k = 0; k < TAPS; ++k) load8(w + (size_t)c * TAPS + k * 8, wv[k]);
            if (bias) load8(bias + c, acc);
            else
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = bias ? to_f32<TW>(bias[c + e]) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < (TAPS > 0 ? TAPS : taps); ++j) {
            const int back = taps - 1 - j;
            const int q = p - back;
            if (q < 0) continue;
            float v[8];
            const bool here = back == 0 || (n - back >= 0 && (tok_seg ? tok_seg[n - back] == seg : false));
            if (here) {
                load8(u + (size_t)(n - back) * ldu + c, v);
            } else if (slot >= 0) {
                const float* sp = state + (size_t)slot * slot_stride + (size_t)(q % (taps - 1)) * channels + c;
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = sp[e];
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.0f;
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float wt = TAPS > 0 ? wv[(e * (TAPS > 0 ? TAPS : 1) + j) / 8][(e * (TAPS > 0 ? TAPS : 1) + j) % 8]
                                          : to_f32<TW>(w[(size_t)(c + e) * taps + j]);
                acc[e] = fmaf(wt, v[e], acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
        store8(out + (size_t)n * channels + c, acc);
        if (ring && slot >= 0 && taps > 1) {
            float v[8];
            load8(u + (size_t)n * ldu + c, v);
            float* dst = ring + (size_t)slot * slot_stride + (size_t)(p % (taps - 1)) * channels + c;
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] = v[e];
        }
    }
}

ZI_EXPORT int zi_causal_conv_silu(const void* u, int dtype, long long ldu, const void* w, const void* bias, int w_dtype,
                                  float* state, long long slot_stride, const int* slots, const int* tok_seg,
                                  const int* pos, void* out, int n_tokens, int channels, int taps, int update_state,
                                  cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps <= 0) return zi_fail("causal_conv: taps=%d must be positive", taps);
    if (update_state && tok_seg) return zi_fail("causal_conv: only a step of single tokens may update the state on the way");
    float* ring = update_state ? state : nullptr;
    if (n_tokens > 65535) return zi_fail("causal_conv: %d tokens are too many for one launch", n_tokens);
    const size_t align = dtype == ZI_BF16 ? 16 : 32;
    if (channels % 8 == 0 && ldu % 8 == 0 && ((uintptr_t)u % align) == 0 && ((uintptr_t)out % align) == 0) {
        dim3 grid((channels / 8 + 127) / 128, n_tokens);
        const size_t walign = w_dtype == ZI_BF16 ? 16 : 32;
        const bool wvec = ((uintptr_t)w % walign) == 0 && (!bias || ((uintptr_t)bias % walign) == 0);
#define ZI_CONV(TAPS_)                                                                                                            \
        ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {                                                                          \
            causal_conv_silu_vec8_kernel<T, TW, TAPS_><<<grid, 128, 0, stream>>>((const T*)u, ldu, (const TW*)w, (const TW*)bias, state, \
                                                                                 slot_stride, slots, tok_seg, pos, (T*)out, n_tokens, \
                                                                                 channels, taps, ring);                          \
        }););
        if (wvec && taps == 4) { ZI_CONV(4) } else if (wvec && taps == 3) { ZI_CONV(3) } else if (wvec && taps == 2) { ZI_CONV(2) } else { ZI_CONV(0) }
#undef ZI_CONV
        return zi_check_launch("causal_conv_silu");
    }
    dim3 grid((channels + 255) / 256, n_tokens);
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(w_dtype, TW, {
        causal_conv_silu_kernel<T, TW><<<grid, 256, 0, stream>>>((const T*)u, ldu, (const TW*)w, (const TW*)bias, state, slot_stride,
                                                                 slots, tok_seg, pos, (T*)out, n_tokens, channels, taps, ring);
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
// A column's state entries are dealt in blocks of R4 (4, 8 or 16) to L lanes of a warp (L a power of two, L * R4 >= N);
// a thread holds the blocks of CPT (1 or 4) neighbouring columns, so that what it reads of B and C serves all of them:
// per token 2 * R4 values from shared memory (16-byte loads; a lane's block starts R4 + 4 floats after its neighbour's, so
// that the eight lanes of a quarter warp hit different banks) against 3 * CPT * R4 multiply-adds.  Tokens come in
// chunks: B, C, x, the step sizes and the decays of a chunk are put into shared memory by the whole block, then every
// thread walks the chunk.  A column's sum over the lanes: with four columns per thread the lanes first halve what they
// hold twice (two exchanges, then one), so that four lanes end with one column each, then add across the rest.
// State in memory: [heads, vdim, N], a column's entries consecutive.
// ---------------------------------------------------------------------------------------
#define SCAN_CHUNK 16
// Long portions (bfloat16 steps): a segment is cut into stretches of SCAN_STRETCH tokens that run side by side.
//   MODE 1  every stretch from a zero state: its own end state and the product of its decays go to a scratch buffer
//   (zi_ssm_combine)  a segment's stretches in order: start state of stretch k = what the request's slot held, carried
//           through stretches 0 .. k-1; it replaces the stretch's own end state in the scratch buffer; the slot receives
//           the state behind the last stretch
//   MODE 2  every stretch again from its start state, this time with C and the outputs
// MODE 0 is the plain walk of a whole segment from the slot's state (float32 steps, short portions, decode steps): its
// sums have one order whatever the cut.  The stretches' sums are the same sums in another order.
#define SCAN_STRETCH 128

__device__ __forceinline__ float softplus_f32(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }

// Two float32 in one 64-bit register and the packed arithmetic of sm_100 on them: one instruction for two values, each
// rounded as the scalar instruction rounds it.
__device__ __forceinline__ uint64_t f2_pack(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) { uint64_t d; asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b)); return d; }

// Which (segment, tokens) a block of a stretch-wise launch works on: stretch number `id` counted through the segments.
__device__ __forceinline__ bool find_stretch(const int* __restrict__ bounds, int n_segments, int id, int* seg, int* first, int* end) {
    for (int s = 0; s < n_segments; ++s) {
        const int b = bounds[2 * s], e = bounds[2 * s + 1];
        const int k = (e - b + SCAN_STRETCH - 1) / SCAN_STRETCH;
        if (id < k) {
            *seg = s;
            *first = b + id * SCAN_STRETCH;
            *end = *first + SCAN_STRETCH < e ? *first + SCAN_STRETCH : e;
            return true;
        }
        id -= k;
    }
    return false;
}

template <typename T, typename TP, int R4, int CPT, int MODE>
__global__ void __launch_bounds__(256, R4 <= 8 ? 3 : 1)
ssm_scan_kernel(const T* __restrict__ xbc, long long ldx, const T* __restrict__ dt_in, long long ld_dt,
                const TP* __restrict__ dt_bias, const TP* __restrict__ a_log, const TP* __restrict__ d_skip,
                float* __restrict__ state, long long slot_stride, const int* __restrict__ slots,
                const int* __restrict__ bounds, float* __restrict__ y, int heads, int vdim, int N, int groups, int L,
                int n_segments, float* __restrict__ scratch, float* __restrict__ decay_out) {
    extern __shared__ __align__(16) float sm[];
    constexpr int RS = R4 == 4 ? 4 : R4 + 4;          // floats between the blocks of neighbouring lanes
    const int h = blockIdx.y;
    const int warps = blockDim.x >> 5, cpw = (32 / L) * CPT, pc = warps * cpw;       // columns per warp, per block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nl = lane % L, col = warp * cpw + (lane / L) * CPT;                    // first of the thread's columns in the tile
    const int p0 = blockIdx.z * pc + col;
    const int g = h / (heads / groups);
    const int inner = heads * vdim;
    const int row = L * RS;
    int seg = blockIdx.x, first, end;
    if (MODE == 0) {
        first = bounds ? bounds[2 * seg] : seg;
        end = bounds ? bounds[2 * seg + 1] : seg + 1;
    } else if (!find_stretch(bounds, n_segments, blockIdx.x, &seg, &first, &end)) {
        return;
    }
    float* Bs = sm;                                  // [chunk][row]
    float* Cs = Bs + SCAN_CHUNK * row;               // [chunk][row]
    float* xs = Cs + SCAN_CHUNK * row;               // [chunk][pc]
    float* dts = xs + SCAN_CHUNK * pc;               // [chunk]
    float* decs = dts + SCAN_CHUNK;                  // [chunk]
    for (int i = threadIdx.x; i < 2 * SCAN_CHUNK * row; i += blockDim.x) sm[i] = 0.0f;     // entries beyond N stay zero
    const float a_rate = expf(to_f32<TP>(a_log[h])), bias = to_f32<TP>(dt_bias[h]), skip = to_f32<TP>(d_skip[h]);
    uint64_t S[CPT][R4 / 2];                         // pairs of neighbouring entries
    // where this block's state comes from and goes to: the request's slot, or the stretch's place in the scratch buffer
    float* sbase;
    bool vec;
    if (MODE == 0) {
        const int slot = slots[seg];
        sbase = slot >= 0 ? state + (size_t)slot * slot_stride + (size_t)h * vdim * N : nullptr;
        vec = (N & 3) == 0 && (slot_stride & 3) == 0 && ((uintptr_t)state & 15) == 0;
    } else {
        sbase = scratch + ((size_t)blockIdx.x * heads + h) * vdim * N;
        vec = (N & 3) == 0 && ((uintptr_t)scratch & 15) == 0;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const bool live = MODE != 1 && sbase && p0 + c < vdim;
        const float* src = live ? sbase + (size_t)(p0 + c) * N + nl * R4 : nullptr;
#pragma unroll
        for (int r = 0; r < R4; r += 4) {
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (live) {
                if (vec) {
                    if (nl * R4 + r < N) v = *reinterpret_cast<const float4*>(src + r);
                } else {
                    if (nl * R4 + r + 0 < N) v.x = src[r + 0];
                    if (nl * R4 + r + 1 < N) v.y = src[r + 1];
                    if (nl * R4 + r + 2 < N) v.z = src[r + 2];
                    if (nl * R4 + r + 3 < N) v.w = src[r + 3];
                }
            }
            S[c][r / 2] = f2_pack(v.x, v.y);
            S[c][r / 2 + 1] = f2_pack(v.z, v.w);
        }
    }
    // eight values per load where everything is a multiple of eight and aligned for it
    const bool vec8 = (N & 7) == 0 && (pc & 7) == 0 && (vdim & 7) == 0 && (inner & 7) == 0 && (ldx & 7) == 0 &&
                      ((uintptr_t)xbc % (8 * sizeof(T))) == 0;
    float decay_all = 1.0f;
    for (int t0 = first; t0 < end; t0 += SCAN_CHUNK) {
        const int cnt = end - t0 < SCAN_CHUNK ? end - t0 : SCAN_CHUNK;
        __syncthreads();
        if (vec8) {
            // per token: N / 8 pieces of B, as many of C (MODE 1 needs none), pc / 8 of x; all of a round's loads before its stores
            const int nb = N >> 3, per = (MODE == 1 ? nb : 2 * nb) + (pc >> 3), items = cnt * per;
            for (int i0 = threadIdx.x; i0 < items; i0 += 2 * blockDim.x) {
                float v[2][8];
                int at[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int i = i0 + q * blockDim.x;
                    at[q] = -1;
                    if (i < items) {
                        const int t = i / per, k = i - t * per;
                        const T* rowp = xbc + (size_t)(t0 + t) * ldx;
                        if (k < nb) {
                            load8(rowp + inner + (size_t)g * N + k * 8, v[q]);
                            at[q] = t * row + ((k * 8) / R4) * RS + (k * 8) % R4;
                        } else if (MODE != 1 && k < 2 * nb) {
                            load8(rowp + inner + (size_t)(groups + g) * N + (k - nb) * 8, v[q]);
                            at[q] = SCAN_CHUNK * row + t * row + (((k - nb) * 8) / R4) * RS + ((k - nb) * 8) % R4;
                        } else {
                            const int c8 = (k - (MODE == 1 ? nb : 2 * nb)) * 8, pp = blockIdx.z * pc + c8;
                            if (pp < vdim) load8(rowp + (size_t)h * vdim + pp, v[q]);
                            else
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[q][e] = 0.0f;
                            at[q] = 2 * SCAN_CHUNK * row + t * pc + c8;
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    if (at[q] >= 0) {
                        // eight values lie in one block of R4 = 8 or 16, or in two blocks of 4
                        *reinterpret_cast<float4*>(sm + at[q]) = make_float4(v[q][0], v[q][1], v[q][2], v[q][3]);
                        const int second = (R4 == 4 && at[q] < 2 * SCAN_CHUNK * row) ? at[q] + RS : at[q] + 4;
                        *reinterpret_cast<float4*>(sm + second) = make_float4(v[q][4], v[q][5], v[q][6], v[q][7]);
                    }
            }
        } else {
            for (int t = warp; t < cnt; t += warps) {
                const T* src = xbc + (size_t)(t0 + t) * ldx + inner + (size_t)g * N;
                for (int n = lane; n < N; n += 32) {
                    const int at = t * row + (n / R4) * RS + (n % R4);
                    Bs[at] = to_f32<T>(src[n]);
                    if (MODE != 1) Cs[at] = to_f32<T>(src[(size_t)groups * N + n]);
                }
                const T* xsrc = xbc + (size_t)(t0 + t) * ldx + (size_t)h * vdim + blockIdx.z * pc;
                for (int c = lane; c < pc; c += 32) xs[t * pc + c] = blockIdx.z * pc + c < vdim ? to_f32<T>(xsrc[c]) : 0.0f;
            }
        }
        for (int t = threadIdx.x; t < cnt; t += blockDim.x) {
            const float dt = softplus_f32(to_f32<T>(dt_in[(size_t)(t0 + t) * ld_dt + h]) + bias);
            dts[t] = dt;
            decs[t] = expf(-a_rate * dt);
        }
        __syncthreads();
        for (int t = 0; t < cnt; ++t) {
            const float a = decs[t], dt = dts[t];
            if (MODE == 1) decay_all *= a;
            float xv[CPT], acc[CPT];
            uint64_t dx2[CPT], acc2[CPT];
            const uint64_t a2 = f2_pack(a, a);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                xv[c] = xs[t * pc + col + c];
                const float dx = dt * xv[c];
                dx2[c] = f2_pack(dx, dx);
                acc2[c] = 0ull;
            }
            const float* bt = Bs + t * row + nl * RS;
            const float* ct = Cs + t * row + nl * RS;
            // entries 2i and 2i + 1 of a block go through the packed instructions side by side; a column's sum over the block
            // is (the even entries in order) + (the odd entries in order)
#pragma unroll
            for (int r = 0; r < R4; r += 4) {
                const ulonglong2 b4 = *reinterpret_cast<const ulonglong2*>(bt + r);
                if (MODE == 1) {
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        S[c][r / 2] = f2_fma(dx2[c], b4.x, f2_mul(a2, S[c][r / 2]));
                        S[c][r / 2 + 1] = f2_fma(dx2[c], b4.y, f2_mul(a2, S[c][r / 2 + 1]));
                    }
                    continue;
                }
                const ulonglong2 c4 = *reinterpret_cast<const ulonglong2*>(ct + r);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    S[c][r / 2] = f2_fma(dx2[c], b4.x, f2_mul(a2, S[c][r / 2]));
                    acc2[c] = f2_fma(S[c][r / 2], c4.x, acc2[c]);
                    S[c][r / 2 + 1] = f2_fma(dx2[c], b4.y, f2_mul(a2, S[c][r / 2 + 1]));
                    acc2[c] = f2_fma(S[c][r / 2 + 1], c4.y, acc2[c]);
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float lo, hi;
                f2_unpack(acc2[c], lo, hi);
                acc[c] = lo + hi;
            }
            if (MODE == 1) continue;
            if (CPT == 4 && L >= 4) {
                // lanes halve what they hold: after two exchanges lane (nl & 3) holds column ((nl & 1) ? 2 : 0) + ((nl & 2) ? 1 : 0);
                // every column's sum is the same tree over the lanes as the plain exchange below makes
                const bool hi = lane & 1, hi2 = lane & 2;
                const float r0 = __shfl_xor_sync(0xffffffffu, hi ? acc[0] : acc[CPT > 2 ? 2 : 0], 1);
                const float r1 = __shfl_xor_sync(0xffffffffu, hi ? acc[CPT > 1 ? 1 : 0] : acc[CPT > 3 ? 3 : 0], 1);
                const float k0 = (hi ? acc[CPT > 2 ? 2 : 0] : acc[0]) + r0, k1 = (hi ? acc[CPT > 3 ? 3 : 0] : acc[CPT > 1 ? 1 : 0]) + r1;
                float keep = (hi2 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, hi2 ? k0 : k1, 2);
                for (int o = 4; o < L; o <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
                const int c = (hi ? 2 : 0) + (hi2 ? 1 : 0);
                if (nl < 4 && p0 + c < vdim) {
                    const float xc = c == 0 ? xv[0] : (c == 1 ? xv[CPT > 1 ? 1 : 0] : (c == 2 ? xv[CPT > 2 ? 2 : 0] : xv[CPT > 3 ? 3 : 0]));
                    y[(size_t)(t0 + t) * inner + (size_t)h * vdim + p0 + c] = fmaf(skip, xc, keep);
                }
            } else {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    float v = acc[c];
                    for (int o = 1; o < L; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (nl == 0 && p0 + c < vdim) y[(size_t)(t0 + t) * inner + (size_t)h * vdim + p0 + c] = fmaf(skip, xv[c], v);
                }
            }
        }
    }
    if (MODE == 2) return;
    if (MODE == 1 && threadIdx.x == 0 && blockIdx.z == 0) decay_out[(size_t)blockIdx.x * heads + h] = decay_all;
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        if (!(sbase && p0 + c < vdim)) continue;
        float* dst = sbase + (size_t)(p0 + c) * N + nl * R4;
#pragma unroll
        for (int r = 0; r < R4; r += 4) {
            float e4[4];
            f2_unpack(S[c][r / 2], e4[0], e4[1]);
            f2_unpack(S[c][r / 2 + 1], e4[2], e4[3]);
            if (vec) {
                if (nl * R4 + r < N) *reinterpret_cast<float4*>(dst + r) = make_float4(e4[0], e4[1], e4[2], e4[3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (nl * R4 + r + e < N) dst[r + e] = e4[e];
            }
        }
    }
}

// A segment's stretches in order, one thread per state entry: the start state of every stretch replaces its own end state
// in the scratch buffer, and the slot receives the state behind the last one.
__global__ void ssm_combine_kernel(float* __restrict__ scratch, const float* __restrict__ decay, float* __restrict__ state,
                                   long long slot_stride, const int* __restrict__ slots, const int* __restrict__ bounds,
                                   int n_segments, int heads, int per_head) {
    const int seg = blockIdx.y;
    const int slot = slots[seg];
    int id0 = 0;
    for (int s = 0; s < seg; ++s) id0 += (bounds[2 * s + 1] - bounds[2 * s] + SCAN_STRETCH - 1) / SCAN_STRETCH;
    const int k = (bounds[2 * seg + 1] - bounds[2 * seg] + SCAN_STRETCH - 1) / SCAN_STRETCH;
    const size_t all = (size_t)heads * per_head;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < all; i += (size_t)gridDim.x * blockDim.x) {
        const int h = (int)(i / per_head);
        float run = slot >= 0 ? state[(size_t)slot * slot_stride + i] : 0.0f;
        // eight stretches at a time: their end states and decays are asked for together, then carried through in order
        for (int j0 = 0; j0 < k; j0 += 8) {
            float own[8], dec[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (j0 + q < k) {
                    own[q] = __ldcg(scratch + (size_t)(id0 + j0 + q) * all + i);
                    dec[q] = __ldcg(decay + (size_t)(id0 + j0 + q) * heads + h);
                }
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (j0 + q < k) {
                    scratch[(size_t)(id0 + j0 + q) * all + i] = run;
                    run = fmaf(dec[q], run, own[q]);
                }
        }
        if (slot >= 0 && k > 0) state[(size_t)slot * slot_stride + i] = run;
    }
}

template <typename T, typename TP, int R4, int CPT>
static int ssm_scan_launch(const void* xbc, long long ldx, const void* dt_in, long long ld_dt, const void* dt_bias, const void* a_log,
                           const void* d_skip, float* state, long long slot_stride, const int* slots, const int* bounds, float* y,
                           int n_segments, int heads, int vdim, int N, int groups, int L, int stretches, float* scratch,
                           cudaStream_t stream) {
    constexpr int RS = R4 == 4 ? 4 : R4 + 4;
    const int cpw = (32 / L) * CPT;
    int warps = (vdim + cpw - 1) / cpw;
    if (warps > 8) warps = 8;
    const int pc = warps * cpw;
    const int ptiles = (vdim + pc - 1) / pc;
    const size_t smem = (size_t)SCAN_CHUNK * (2 * L * RS + pc + 2) * sizeof(float);
    if (heads > 65535 || ptiles > 65535) return zi_fail("ssm_scan: too many heads or columns for one launch");
    if (smem > 200 * 1024) return zi_fail("ssm_scan: %zu bytes of shared memory", smem);
#define ZI_SCAN_GO(MODE_, GRIDX_)                                                                                              \
    {                                                                                                                          \
        auto fn = ssm_scan_kernel<T, TP, R4, CPT, MODE_>;                                                                      \
        if (smem > 48 * 1024 && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return zi_fail("ssm_scan: cannot reserve %zu bytes of shared memory", smem);                                       \
        fn<<<dim3(GRIDX_, heads, ptiles), warps * 32, smem, stream>>>((const T*)xbc, ldx, (const T*)dt_in, ld_dt, (const TP*)dt_bias, \
                                                                      (const TP*)a_log, (const TP*)d_skip, state, slot_stride, slots, \
                                                                      bounds, y, heads, vdim, N, groups, L, n_segments, scratch, decay); \
    }
    float* decay = scratch ? scratch + (size_t)stretches * heads * vdim * N : nullptr;
    if (!scratch) {
        ZI_SCAN_GO(0, n_segments)
        return zi_check_launch("ssm_scan");
    }
    ZI_SCAN_GO(1, stretches)
    const size_t all = (size_t)heads * vdim * N;
    const int cb = (int)((all + 255) / 256 > 1024 ? 1024 : (all + 255) / 256);
    ssm_combine_kernel<<<dim3(cb, n_segments), 256, 0, stream>>>(scratch, decay, state, slot_stride, slots, bounds, n_segments, heads,
                                                                 vdim * N);
    ZI_SCAN_GO(2, stretches)
#undef ZI_SCAN_GO
    return zi_check_launch("ssm_scan");
}

// How many stretches a step of n_tokens tokens in n_segments segments has at most, and the floats of scratch that the
// stretch-wise form needs for them (states, then decay products).
ZI_EXPORT int zi_ssm_scan_stretches(int n_tokens, int n_segments) { return n_tokens / SCAN_STRETCH + n_segments; }
ZI_EXPORT long long zi_ssm_scan_scratch_floats(int n_tokens, int n_segments, int heads, int vdim, int N) {
    return (long long)zi_ssm_scan_stretches(n_tokens, n_segments) * heads * ((long long)vdim * N + 1);
}

// scratch: null for the plain walk; else a buffer of zi_ssm_scan_scratch_floats(...) floats, and every segment's stretches
// run side by side (bounds required).
ZI_EXPORT int zi_ssm_scan(const void* xbc, int dtype, long long ldx, const void* dt_in, long long ld_dt, const void* dt_bias,
                          const void* a_log, const void* d_skip, int p_dtype, float* state, long long slot_stride,
                          const int* slots, const int* bounds, float* y, int n_tokens, int n_segments, int heads, int vdim, int N,
                          int groups, float* scratch, cudaStream_t stream) {
    if (n_segments <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || N <= 0 || groups <= 0 || heads % groups)
        return zi_fail("ssm_scan: heads=%d vdim=%d state=%d groups=%d", heads, vdim, N, groups);
    if (N > 512) return zi_fail("ssm_scan: state=%d is more than 512", N);
    if (scratch && !bounds) return zi_fail("ssm_scan: the stretch-wise form needs the segments' bounds");
    const int stretches = zi_ssm_scan_stretches(n_tokens, n_segments);
    // the state's entries: blocks of 8 on as few lanes as take them (blocks of 16 beyond 256 entries, of 4 up to 4)
    const int r4 = N > 256 ? 16 : (N <= 4 ? 4 : 8);
    int L = 1;
    while (L * r4 < N) L *= 2;
    const int cpt = vdim >= 4 ? 4 : 1;
#define ZI_SCAN(R4_, CPT_) \
    ZI_DISPATCH(dtype, T, ZI_DISPATCH(p_dtype, TP, { \
        return ssm_scan_launch<T, TP, R4_, CPT_>(xbc, ldx, dt_in, ld_dt, dt_bias, a_log, d_skip, state, slot_stride, slots, bounds, y, \
                                                 n_segments, heads, vdim, N, groups, L, stretches, scratch, stream); }););
    if (cpt == 4) {
        if (r4 == 4) { ZI_SCAN(4, 4) } else if (r4 == 8) { ZI_SCAN(8, 4) } else { ZI_SCAN(16, 4) }
    } else {
        if (r4 == 4) { ZI_SCAN(4, 1) } else if (r4 == 8) { ZI_SCAN(8, 1) } else { ZI_SCAN(16, 1) }
    }
#undef ZI_SCAN
    return zi_fail("ssm_scan: no kernel for these sizes");
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
