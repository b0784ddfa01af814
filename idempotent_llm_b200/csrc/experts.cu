// Feed-forward experts chosen per token: out[t] = weight * sum_k down_e (act(gate_e x_t) * up_e x_t), e = the
// k-th expert of token t = table[token id of t, k] (a table of integers [vocabulary, top]).  These kernels serve steps of few tokens (single tokens above all): every (token,
// choice) streams its expert's matrices once, a warp per output row, sums in 32-bit in a fixed order, so a
// token's result does not depend on what else the step holds.  Steps of many tokens group their rows by expert
// on the host and run one matrix product per expert instead; the kernels below then gather the rows
// (rows_gather) and add the experts' outputs back in the order of a token's choices (experts_combine).
//
// A learned router names a token's experts on the device: then `tokens` holds the step's row numbers and `table` the
// step's choices [rows, top], and `pair_w` [rows, top] (null: 1) is the weight of every (token, choice) beside the
// constant `weight`.  Where an expert's activations are 32-bit numbers of these kernels' own, the pair's weight is
// multiplied into them (the down product is linear); where the library's products make them, the weight is applied
// when the experts' outputs are added.
#include "common.cuh"

__device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ xs, int K, int lane, bool vec) {
    float s = 0.f;
    if (vec) {
        constexpr int VN = Vec16<T>::N;
        for (int d = lane * VN; d < K; d += 32 * VN) {
            Vec16<T> wv; wv.load(w + d);
#pragma unroll
            for (int e = 0; e < VN; ++e) s = fmaf(xs[d + e], wv.get(e), s);
        }
    } else {
        for (int d = lane; d < K; d += 32) s = fmaf(xs[d], to_f32(w[d]), s);
    }
    return warp_sum(s);
}

// two rows against two vectors at once: eight (long rows) or four 16-byte loads of a lane are in flight before the
// first is used; a sum's order depends on the row's length alone
__device__ __forceinline__ void row_dot2(const T* __restrict__ w0, const T* __restrict__ w1, const float* __restrict__ x0,
                                         const float* __restrict__ x1, int K, int lane, bool vec, float& r0, float& r1) {
    float s0 = 0.f, s1 = 0.f;
    if (vec) {
        constexpr int VN = Vec16<T>::N;
        int d = lane * VN;
        for (; d + 96 * VN < K; d += 128 * VN) {             // four pieces of each row: eight loads before the first use
            Vec16<T> a[4], b[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) { a[c].load(w0 + d + c * 32 * VN); b[c].load(w1 + d + c * 32 * VN); }
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    s0 = fmaf(x0[d + c * 32 * VN + e], a[c].get(e), s0);
                    s1 = fmaf(x1[d + c * 32 * VN + e], b[c].get(e), s1);
                }
        }
        for (; d + 32 * VN < K; d += 64 * VN) {
            Vec16<T> a0, a1, b0, b1;
            a0.load(w0 + d); b0.load(w1 + d); a1.load(w0 + d + 32 * VN); b1.load(w1 + d + 32 * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) { s0 = fmaf(x0[d + e], a0.get(e), s0); s1 = fmaf(x1[d + e], b0.get(e), s1); }
#pragma unroll
            for (int e = 0; e < VN; ++e) { s0 = fmaf(x0[d + 32 * VN + e], a1.get(e), s0); s1 = fmaf(x1[d + 32 * VN + e], b1.get(e), s1); }
        }
        for (; d < K; d += 32 * VN) {
            Vec16<T> a0, b0;
            a0.load(w0 + d); b0.load(w1 + d);
#pragma unroll
            for (int e = 0; e < VN; ++e) { s0 = fmaf(x0[d + e], a0.get(e), s0); s1 = fmaf(x1[d + e], b0.get(e), s1); }
        }
    } else {
        for (int d = lane; d < K; d += 32) { s0 = fmaf(x0[d], to_f32(w0[d]), s0); s1 = fmaf(x1[d], to_f32(w1[d]), s1); }
    }
    r0 = warp_sum(s0); r1 = warp_sum(s1);
}

// a[t, k, f] = act(gate_e[f] . x_t) * (up_e[f] . x_t), 32-bit.  Gate and up rows of an expert lie in one array:
// row f of expert e starts at e * expert_stride + f * row_stride (gate) and up_off behind that (up), which serves both
// "gate rows, then up rows" and "gate and up rows alternating" (the layout a gated product's epilogue reads).
// A block has one (token, choice) and 8 rows f per pass of its warps.
__global__ void __launch_bounds__(256) experts_gate_up_kernel(const T* __restrict__ x, const int* __restrict__ tokens,
                                                              const int* __restrict__ table, const float* __restrict__ pair_w,
                                                              const T* __restrict__ gate_up, long long expert_stride,
                                                              long long row_stride, long long up_off,
                                                              float* __restrict__ a, int width, int ff, int top, int n_experts,
                                                              int act) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];
    const int tk = blockIdx.x;
    const int t = tk / top;
    const int e = table[(size_t)tokens[t] * top + tk % top];       // the token's id names its experts
    for (int d = threadIdx.x; d < width; d += blockDim.x) xs[d] = to_f32(x[(size_t)t * width + d]);
    __syncthreads();
    if (e < 0 || e >= n_experts) return;                     // (a table entry outside the experts: contributes nothing)
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (width * (int)sizeof(T)) % 16 == 0;
    const float pw = pair_w ? pair_w[tk] : 1.f;
    for (int f = blockIdx.y * 8 + wib; f < ff; f += gridDim.y * 8) {
        const T* row = gate_up + (size_t)e * expert_stride + (size_t)f * row_stride;
        float g, u;
        row_dot2(row, row + up_off, xs, xs, width, lane, vec, g, u);
        if (lane == 0) a[(size_t)tk * ff + f] = pair_w ? gated_act(g, u, act) * pw : gated_act(g, u, act);
    }
}

// h[t, w] += weight * sum_k down_e[w] . a[t, k];  down: [E, width, ff]; a block has one token, a warp an output row
__global__ void __launch_bounds__(256) experts_down_kernel(const float* __restrict__ a, const int* __restrict__ tokens,
                                                           const int* __restrict__ table,
                                                           const T* __restrict__ down, float* __restrict__ h, int width,
                                                           int ff, int top, int n_experts, float weight) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float as[];                             // [top][ff]
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < top * ff; d += blockDim.x) as[d] = a[(size_t)t * top * ff + d];
    __syncthreads();
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (ff * (int)sizeof(T)) % 16 == 0;
    for (int w = blockIdx.y * 8 + wib; w < width; w += gridDim.y * 8) {
        float s = 0.f;
        int k = 0;
        for (; k + 1 < top; k += 2) {                       // two choices' rows at once (their loads side by side)
            const int e0 = table[(size_t)tokens[t] * top + k], e1 = table[(size_t)tokens[t] * top + k + 1];
            const bool ok0 = e0 >= 0 && e0 < n_experts, ok1 = e1 >= 0 && e1 < n_experts;
            if (ok0 && ok1) {
                float r0, r1;
                row_dot2(down + ((size_t)e0 * width + w) * ff, down + ((size_t)e1 * width + w) * ff, as + k * ff, as + (k + 1) * ff,
                         ff, lane, vec, r0, r1);
                s += r0; s += r1;
            } else {
                if (ok0) s += row_dot(down + ((size_t)e0 * width + w) * ff, as + k * ff, ff, lane, vec);
                if (ok1) s += row_dot(down + ((size_t)e1 * width + w) * ff, as + (k + 1) * ff, ff, lane, vec);
            }
        }
        for (; k < top; ++k) {
            const int e = table[(size_t)tokens[t] * top + k];
            if (e < 0 || e >= n_experts) continue;
            s += row_dot(down + ((size_t)e * width + w) * ff, as + k * ff, ff, lane, vec);
        }
        if (lane == 0) h[(size_t)t * width + w] += s * weight;
    }
}

extern "C" int idm_experts_few(const void* x, const int* tokens, const int* table, const float* pair_w, const void* gate_up, long long expert_stride,
                               long long row_stride, long long up_off, const void* down,
                               float* a, float* h, int n_tokens, int width, int ff, int top, int n_experts, int act,
                               float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && ff > 0 && top > 0 && n_experts > 0 && (act >= 0 && act <= 2), "experts: width=%d ff=%d top=%d experts=%d act=%d",
                width, ff, top, n_experts, act);
    IDM_REQUIRE((size_t)width * 4 <= 160 * 1024 && (size_t)top * ff * 4 <= 160 * 1024, "experts: width=%d or top * ff=%d does not fit shared memory",
                width, top * ff);
    const size_t s1 = (size_t)width * 4, s2 = (size_t)top * ff * 4;
    if (s1 > 48 * 1024) cudaFuncSetAttribute(experts_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    if (s2 > 48 * 1024) cudaFuncSetAttribute(experts_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2);
    // blocks along the rows: enough to fill the part for one token, fewer per token as tokens grow
    const int by1 = max(1, min((ff + 7) / 8, 592 / max(1, n_tokens * top)));
    const int by2 = max(1, min((width + 7) / 8, 592 / max(1, n_tokens)));
    idm_launch(experts_gate_up_kernel, dim3(n_tokens * top, by1), dim3(256), s1, stream, (const T*)x, tokens, table, pair_w, (const T*)gate_up,
               expert_stride, row_stride, up_off, a, width, ff, top, n_experts, act);
    IDM_LAUNCH_CHECK("experts_gate_up");
    idm_launch(experts_down_kernel, dim3(n_tokens, by2), dim3(256), s2, stream, (const float*)a, tokens, table, (const T*)down, h, width,
               ff, top, n_experts, weight);
    IDM_LAUNCH_CHECK("experts_down");
    return 0;
}

// out[i, :] = x[src[i], :]  (rows of the storage type; a step's rows in the order of their experts)
__global__ void __launch_bounds__(256) rows_gather_kernel(const T* __restrict__ x, const int* __restrict__ src, T* __restrict__ out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = blockIdx.x;
    const T* r = x + (size_t)src[i] * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) out[i * width + d] = r[d];
}

extern "C" int idm_rows_gather(const void* x, const int* src, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    idm_launch(rows_gather_kernel, dim3(n_rows), dim3(256), 0, stream, (const T*)x, src, (T*)out, width);
    IDM_LAUNCH_CHECK("rows_gather");
    return 0;
}

// h[t, :] += weight * sum_k z[place[t, k], :] in ascending k  (z 32-bit: the experts' outputs, grouped rows)
__global__ void __launch_bounds__(256) experts_combine_kernel(const float* __restrict__ z, const int* __restrict__ place,
                                                              const float* __restrict__ pair_w, float* __restrict__ h, int width,
                                                              int top, float weight) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int r = place ? place[t * top + k] : (int)(t * top + k);      // (no places: pair by pair as they lie)
            if (r >= 0) s = pair_w ? fmaf(pair_w[t * top + k], z[(size_t)r * width + d], s) : s + z[(size_t)r * width + d];
        }
        h[t * width + d] += s * weight;
    }
}

extern "C" int idm_experts_combine(const float* z, const int* place, const float* pair_w, float* h, int n_tokens, int width,
                                   int top, float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    idm_launch(experts_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, z, place, pair_w, h, width, top, weight);
    IDM_LAUNCH_CHECK("experts_combine");
    return 0;
}

// ------------------------------------------------------------------ the same, expert by expert
// For steps of more than a few tokens whose ids exist on the device only: a block has one expert and a slice of its
// rows, finds the (token, choice) pairs that use the expert (in ascending order), and walks them eight at a time: the
// eight input vectors wait in shared memory, a warp streams a row of the expert's matrix once for all eight.  An expert
// is read from memory once a step however many tokens use it.  MODE 0: a[pair, f] = act(gate[f] . x_t) * (up[f] . x_t);
// MODE 1: z[pair, w] = down[w] . a[pair].  Sums in 32-bit, lanes over the inner axis, then a butterfly.
#define EX_TOKENS 8

template <int MODE>
__global__ void __launch_bounds__(256) experts_major_kernel(const T* __restrict__ x, const float* __restrict__ a_in,
                                                            const int* __restrict__ tokens, const int* __restrict__ table,
                                                            const float* __restrict__ pair_w,
                                                            const T* __restrict__ w, long long expert_stride, long long row_stride,
                                                            long long up_off, float* __restrict__ out, int n_tokens, int top,
                                                            int K, int rows, int act) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    float* xs = sm;                                              // [EX_TOKENS][K]
    int* pairs = reinterpret_cast<int*>(sm + EX_TOKENS * K);     // [n_tokens * top]
    __shared__ int count_s;
    const int e = blockIdx.x, wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (wib == 0) {                                              // the pairs of this expert, in ascending order
        int count = 0;
        for (int p0 = 0; p0 < n_tokens * top; p0 += 32) {
            const int p = p0 + lane;
            const bool mine = p < n_tokens * top && table[(size_t)tokens[p / top] * top + p % top] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) pairs[count + __popc(m & ((1u << lane) - 1u))] = p;
            count += __popc(m);
        }
        if (lane == 0) count_s = count;
    }
    __syncthreads();
    const int count = count_s;
    if (count == 0) return;
    const bool vec = (K * (int)sizeof(T)) % 16 == 0;
    const T* we = w + (size_t)e * expert_stride;
    for (int p0 = 0; p0 < count; p0 += EX_TOKENS) {
        const int np = min(EX_TOKENS, count - p0);
        __syncthreads();                                         // the last eight's readers are done
        for (int i = threadIdx.x; i < EX_TOKENS * K; i += blockDim.x) {
            const int tt = i / K, d = i % K;
            float v = 0.f;
            if (tt < np) {
                const int p = pairs[p0 + tt];
                v = MODE == 0 ? to_f32(x[(size_t)(p / top) * K + d]) : a_in[(size_t)p * K + d];
            }
            xs[i] = v;
        }
        __syncthreads();
        for (int r = blockIdx.y * 8 + wib; r < rows; r += gridDim.y * 8) {
            const T* w0 = we + (size_t)r * row_stride;
            float g[EX_TOKENS], u[EX_TOKENS];
#pragma unroll
            for (int tt = 0; tt < EX_TOKENS; ++tt) g[tt] = u[tt] = 0.f;
            if (vec) {
                constexpr int VN = Vec16<T>::N;
                // four 16-byte pieces of the row (and of its partner) per lane are requested before the first is used
                for (int d0 = lane * VN; d0 < K; d0 += 4 * 32 * VN) {
                    Vec16<T> wg[4], wu[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int d = d0 + c * 32 * VN;
                        if (d < K) {
                            wg[c].load(w0 + d);
                            if (MODE == 0) wu[c].load(w0 + up_off + d);
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int d = d0 + c * 32 * VN;
                        if (d < K) {
#pragma unroll
                            for (int tt = 0; tt < EX_TOKENS; ++tt) {
#pragma unroll
                                for (int q = 0; q < VN; q += 4) {
                                    const float4 xv = *reinterpret_cast<const float4*>(xs + tt * K + d + q);
                                    g[tt] = fmaf(xv.x, wg[c].get(q), g[tt]); g[tt] = fmaf(xv.y, wg[c].get(q + 1), g[tt]);
                                    g[tt] = fmaf(xv.z, wg[c].get(q + 2), g[tt]); g[tt] = fmaf(xv.w, wg[c].get(q + 3), g[tt]);
                                    if (MODE == 0) {
                                        u[tt] = fmaf(xv.x, wu[c].get(q), u[tt]); u[tt] = fmaf(xv.y, wu[c].get(q + 1), u[tt]);
                                        u[tt] = fmaf(xv.z, wu[c].get(q + 2), u[tt]); u[tt] = fmaf(xv.w, wu[c].get(q + 3), u[tt]);
                                    }
                                }
                            }
                        }
                    }
                }
            } else {
                for (int d = lane; d < K; d += 32) {
                    const float wg = to_f32(w0[d]), wu = MODE == 0 ? to_f32(w0[up_off + d]) : 0.f;
#pragma unroll
                    for (int tt = 0; tt < EX_TOKENS; ++tt) {
                        g[tt] = fmaf(xs[tt * K + d], wg, g[tt]);
                        if (MODE == 0) u[tt] = fmaf(xs[tt * K + d], wu, u[tt]);
                    }
                }
            }
#pragma unroll
            for (int tt = 0; tt < EX_TOKENS; ++tt) {
                g[tt] = warp_sum(g[tt]);
                if (MODE == 0) u[tt] = warp_sum(u[tt]);
            }
            if (lane == 0) {
#pragma unroll
                for (int tt = 0; tt < EX_TOKENS; ++tt)
                    if (tt < np) {
                        const int pr = pairs[p0 + tt];
                        out[(size_t)pr * rows + r] = MODE == 0 ? (pair_w ? gated_act(g[tt], u[tt], act) * pair_w[pr] : gated_act(g[tt], u[tt], act)) : g[tt];
                    }
            }
        }
    }
}

// z: [n_tokens * top, width] 32-bit scratch for the experts' outputs (then added to h pair by pair in ascending k)
extern "C" int idm_experts_major(const void* x, const int* tokens, const int* table, const float* pair_w, const void* gate_up,
                                 long long expert_stride, long long row_stride, long long up_off, const void* down,
                                 float* a, float* z, float* h, int n_tokens, int width, int ff, int top, int n_experts,
                                 int act, float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && ff > 0 && top > 0 && n_experts > 0 && (act >= 0 && act <= 2), "experts: width=%d ff=%d top=%d experts=%d act=%d",
                width, ff, top, n_experts, act);
    const size_t s1 = (size_t)EX_TOKENS * width * 4 + (size_t)n_tokens * top * 4, s2 = (size_t)EX_TOKENS * ff * 4 + (size_t)n_tokens * top * 4;
    IDM_REQUIRE(s1 <= 200 * 1024 && s2 <= 200 * 1024, "experts: width=%d or ff=%d with %d tokens does not fit shared memory", width, ff, n_tokens);
    if (s1 > 48 * 1024) cudaFuncSetAttribute(experts_major_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    if (s2 > 48 * 1024) cudaFuncSetAttribute(experts_major_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2);
    const int by1 = max(1, min((ff + 7) / 8, 592 / n_experts)), by2 = max(1, min((width + 7) / 8, 592 / n_experts));
    idm_launch(experts_major_kernel<0>, dim3(n_experts, by1), dim3(256), s1, stream, (const T*)x, (const float*)nullptr, tokens, table, pair_w,
               (const T*)gate_up, expert_stride, row_stride, up_off, a, n_tokens, top, width, ff, act);
    IDM_LAUNCH_CHECK("experts_major gate/up");
    idm_launch(experts_major_kernel<1>, dim3(n_experts, by2), dim3(256), s2, stream, (const T*)nullptr, (const float*)a, tokens, table, (const float*)nullptr,
               (const T*)down, (long long)width * ff, (long long)ff, 0LL, z, n_tokens, top, ff, width, act);
    IDM_LAUNCH_CHECK("experts_major down");
    idm_launch(experts_combine_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)z, (const int*)nullptr, (const float*)nullptr, h,
               width, top, weight);
    IDM_LAUNCH_CHECK("experts_combine");
    return 0;
}

#if defined(IDM_BF16)
// Every expert's gated feed-forward over its slice of rows grouped by expert: the library's own matrix products (the
// gate/up product with the activation as its epilogue, then the down product), expert after expert, from one call.
// counts: on the HOST, rows of each expert; gate_up [E, tiles * 128, width] alternating rows; down [E, width, ff].
extern "C" int idm_gemm_bf16_gated(const void* x, const void* w, void* y, int M, int inter, int K, int act, cudaStream_t stream);
extern "C" int idm_gemm_bf16(const void* x, const void* w, float* out, int M, int N, int K, cudaStream_t stream);

extern "C" int idm_experts_grouped(const void* xg, const int* counts, int n_experts, const void* gate_up,
                                   long long gate_up_stride, const void* down, long long down_stride, void* y, float* z,
                                   int width, int ff, int act, cudaStream_t stream) {
    IDM_REQUIRE(width > 0 && ff > 0 && width % 8 == 0 && ff % 8 == 0, "experts_grouped: width=%d ff=%d (multiples of 8)", width, ff);
    long long at = 0;
    for (int e = 0; e < n_experts; ++e) {
        const int c = counts[e];
        if (c <= 0) continue;
        const T* xe = (const T*)xg + at * width;
        T* ye = (T*)y + at * ff;
        if (idm_gemm_bf16_gated(xe, (const T*)gate_up + (long long)e * gate_up_stride, ye, c, ff, width, act, stream)) return 1;
        if (idm_gemm_bf16(ye, (const T*)down + (long long)e * down_stride, z + at * width, c, width, ff, stream)) return 1;
        at += c;
    }
    return 0;
}

// The grouped feed-forward of a step from one call: rows gathered in the order of their experts (src: grouped row ->
// token), every expert's two products, outputs added into the stream in the order of a token's choices (place:
// (token, choice) -> grouped row).  xg, y, z: scratch [n_tokens * top, width | ff | width].
extern "C" int idm_experts_grouped_step(const void* x, const int* src, const int* place, const float* pair_w, const int* counts, int n_experts,
                                        const void* gate_up, long long gate_up_stride, const void* down, long long down_stride,
                                        void* xg, void* y, float* z, float* h, int n_tokens, int top, int width, int ff, int act,
                                        float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    if (idm_rows_gather(x, src, xg, n_tokens * top, width, stream)) return 1;
    if (idm_experts_grouped(xg, counts, n_experts, gate_up, gate_up_stride, down, down_stride, y, z, width, ff, act, stream)) return 1;
    return idm_experts_combine(z, place, pair_w, h, n_tokens, width, top, weight, stream);
}

// Single-token steps of many sequences, whose ids exist on the device only and whose shapes must not change from
// step to step: EVERY expert's feed-forward over ALL the step's tokens with the library's matrix products (what such a
// step has to do anyway is to stream every expert's matrices once: the products it does not need ride along), then
// each token takes the outputs of its own experts.  z_all: [E, n_tokens, width] 32-bit; y: [n_tokens, ff] scratch.
__global__ void __launch_bounds__(256) experts_pick_kernel(const float* __restrict__ z_all, const int* __restrict__ tokens,
                                                           const int* __restrict__ table, const float* __restrict__ pair_w,
                                                           float* __restrict__ h, int n_tokens, int width, int top, int n_experts,
                                                           float weight) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = table[(size_t)tokens[t] * top + k];
            if (e >= 0 && e < n_experts) {
                const float z = z_all[((size_t)e * n_tokens + t) * width + d];
                s = pair_w ? fmaf(pair_w[t * top + k], z, s) : s + z;
            }
        }
        h[t * width + d] += s * weight;
    }
}

extern "C" int idm_experts_dense(const void* x, const int* tokens, const int* table, const float* pair_w, int n_experts, const void* gate_up,
                                 long long gate_up_stride, const void* down, long long down_stride, void* y, float* z_all,
                                 float* h, int n_tokens, int width, int ff, int top, int act, float weight, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && ff > 0 && width % 8 == 0 && ff % 8 == 0, "experts_dense: width=%d ff=%d (multiples of 8)", width, ff);
    for (int e = 0; e < n_experts; ++e) {
        if (idm_gemm_bf16_gated(x, (const T*)gate_up + (long long)e * gate_up_stride, y, n_tokens, ff, width, act, stream)) return 1;
        if (idm_gemm_bf16(y, (const T*)down + (long long)e * down_stride, z_all + (size_t)e * n_tokens * width, n_tokens, width, ff, stream)) return 1;
    }
    idm_launch(experts_pick_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)z_all, tokens, table, pair_w, h, n_tokens, width, top,
               n_experts, weight);
    IDM_LAUNCH_CHECK("experts_pick");
    return 0;
}
#endif
