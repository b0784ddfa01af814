// Embedding, residual-add + RMS norm, rotary table, q/k norm + rotation + cache
// write, ring write, SwiGLU.  Memory-bound kernels; everything that follows a
// matrix product reads its 32-bit partial sums and adds them in ascending order.
#include "common.cuh"
#include "qkv_finish.cuh"

// ------------------------------------------------------------------ embedding
// h[t, :] = table[tokens[t], :]  (a pure lookup, no scaling: src/detllm/model.py:246-249)
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ h, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + (size_t)tokens[t] * hidden;
    float* out = h + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32(row[i]);
}

extern "C" int idm_embed(const int* tokens, const void* table, float* h, int n_tokens, int hidden,
                         cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(n_tokens > 0 && hidden > 0, "embed: bad sizes n_tokens=%d hidden=%d", n_tokens, hidden);
    idm_launch(embed_kernel, dim3(n_tokens), dim3(256), 0, stream, tokens, (const T*)table, h, hidden);
    IDM_LAUNCH_CHECK("embed");
    return 0;
}

// ------------------------------------------------------- residual add + RMSNorm
// rows == nullptr: for every token row r: h[r] += sum_p delta[p][r] (stored), x[r] = norm(h[r]).
// rows != nullptr: for i < n_rows: v = h[rows[i]] + sum_p delta[p][rows[i]] (not stored), x[i] = norm(v).
// norm(v) = v / sqrt(mean(v^2) + eps) * gamma, in 32-bit.  One block per row; the block
// size is fixed, so the reduction order depends on `hidden` only.
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                   size_t partial_stride, const float* __restrict__ gamma, float eps,
                                   T* __restrict__ x, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];            // the row, kept between the two passes
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = add_partials(hr[c], delta, n_partials, partial_stride, (size_t)r * hidden + c);
        if (!rows && n_partials) hr[c] = v;
        vals[c] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* xr = x + (size_t)i * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) from_f32(xr[c], vals[c] * inv * gamma[c]);
}

// The same for rows of at most 4 * 256 elements with hidden % 4 == 0: a thread owns four consecutive
// elements, and all of its loads (the stream and up to 16 partials) are in flight at once.
__global__ void __launch_bounds__(256) add_rmsnorm_vec4_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                               int n_partials, size_t partial_stride,
                                                               const float* __restrict__ gamma, float eps,
                                                               T* __restrict__ x, const int* __restrict__ rows,
                                                               int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const int c = threadIdx.x * 4;
    const bool live = c < hidden;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        const size_t idx = (size_t)r * hidden + c;
        v = *reinterpret_cast<const float4*>(h + idx);
        if (n_partials > 0) {
            float4 part[16];
#pragma unroll
            for (int p = 0; p < 16; ++p)
                if (p < n_partials) part[p] = *reinterpret_cast<const float4*>(delta + p * partial_stride + idx);
#pragma unroll
            for (int p = 0; p < 16; ++p)
                if (p < n_partials) { v.x += part[p].x; v.y += part[p].y; v.z += part[p].z; v.w += part[p].w; }
        }
        if (!rows && n_partials) *reinterpret_cast<float4*>(h + idx) = v;
    }
    const float total = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    if (live) {
        const float4 gm = *reinterpret_cast<const float4*>(gamma + c);
        T* xr = x + (size_t)i * hidden + c;
        store4(xr, v.x * inv * gm.x, v.y * inv * gm.y, v.z * inv * gm.z, v.w * inv * gm.w);
    }
}

// Many rows with nothing to add (the residual was added by the product before): one warp per row, no
// block-wide barrier.  Lane l stands for the threads l, l + 32, ... of the kernel above (its warps
// 0 .. 7), sums each of those warps by the same butterfly and adds the eight totals in the same order:
// the same bits, whichever of the two kernels runs.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ h, const float* __restrict__ gamma,
                                                           float eps, T* __restrict__ x, const int* __restrict__ rows,
                                                           int n_rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const int r = rows ? rows[i] : i;
    const float* hr = h + (size_t)r * hidden;
    float4 v[8];
    float s[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        v[w] = c < hidden ? *reinterpret_cast<const float4*>(hr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        s[w] = v[w].x * v[w].x + v[w].y * v[w].y + v[w].z * v[w].z + v[w].w * v[w].w;
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) s[w] = warp_sum(s[w]);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += s[w];
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* xr = x + (size_t)i * hidden;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        if (c < hidden) {
            const float4 gm = *reinterpret_cast<const float4*>(gamma + c);
            store4(xr + c, v[w].x * inv * gm.x, v[w].y * inv * gm.y, v[w].z * inv * gm.z, v[w].w * inv * gm.w);
        }
    }
}

extern "C" int idm_add_rmsnorm(float* h, const float* delta, int n_partials, long long partial_stride,
                               const float* gamma, float eps, void* x, const int* rows, int n_rows,
                               int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "add_rmsnorm: hidden=%d does not fit shared memory", hidden);
    if (hidden % 4 == 0 && hidden <= 1024 && (delta == nullptr || n_partials == 0) && n_rows >= 64) {
        idm_launch(rmsnorm_rows_kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, (const float*)h, gamma, eps, (T*)x, rows,
                   n_rows, hidden);
        IDM_LAUNCH_CHECK("add_rmsnorm");
        return 0;
    }
    if (hidden % 4 == 0 && hidden <= 1024 && n_partials <= 16 && (partial_stride % 4) == 0) {
        // NOTE: the sum of squares is taken over the same values in a different thread layout than
        // the general kernel; which kernel runs depends on `hidden` and the number of partials only
        idm_launch(add_rmsnorm_vec4_kernel, dim3(n_rows), dim3(256), 0, stream, h, delta, delta ? n_partials : 0, (size_t)partial_stride,
                                                            gamma, eps, (T*)x, rows, hidden);
        IDM_LAUNCH_CHECK("add_rmsnorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(add_rmsnorm_kernel, dim3(n_rows), dim3(256), smem, stream, h, delta, delta ? n_partials : 0,
                                                      (size_t)partial_stride, gamma, eps, (T*)x, rows, hidden);
    IDM_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// Two norms of the same row with one pass over it, for layers whose mixer and feed-forward both read the stream
// as it stands: h[r] += sum_p delta[p][r] (stored), x1 = norm(h[r]) * gamma1, x2 = norm(h[r]) * gamma2 (null: the
// layer has no second reader); the root mean square is taken once.  `post`, if given, is a constant row added to
// the stream AFTER the norms are taken (a bias of the layer's output that does not depend on its input), so
// that no pass of its own has to add it.
__global__ void __launch_bounds__(256) add_rmsnorm2_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                           size_t partial_stride, const float* __restrict__ gamma1,
                                                           const float* __restrict__ gamma2, float eps, T* __restrict__ x1,
                                                           T* __restrict__ x2, const float* __restrict__ post, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = add_partials(hr[c], delta, n_partials, partial_stride, (size_t)r * hidden + c);
        if (n_partials || post) hr[c] = post ? v + post[c] : v;
        vals[c] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* xr1 = x1 + (size_t)r * hidden;
    T* xr2 = x2 ? x2 + (size_t)r * hidden : nullptr;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float n = vals[c] * inv;
        from_f32(xr1[c], n * gamma1[c]);
        if (xr2) from_f32(xr2[c], n * gamma2[c]);
    }
}

// The same for rows of at most NV * 1024 elements with hidden % 4 == 0: a thread owns NV pieces of four consecutive
// elements in registers (no staging in shared memory), all of its loads of the stream in flight at once.
template <int NV>
__global__ void __launch_bounds__(256) add_rmsnorm2_vec4_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                                size_t partial_stride, const float* __restrict__ gamma1,
                                                                const float* __restrict__ gamma2, float eps, T* __restrict__ x1,
                                                                T* __restrict__ x2, const float* __restrict__ post, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (threadIdx.x + 256 * k) * 4;
        v[k] = c < hidden ? *reinterpret_cast<const float4*>(h + (size_t)r * hidden + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (threadIdx.x + 256 * k) * 4;
        if (c < hidden) {
            const size_t idx = (size_t)r * hidden + c;
            for (int p = 0; p < n_partials; ++p) {
                const float4 d = *reinterpret_cast<const float4*>(delta + p * partial_stride + idx);
                v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
            }
            if (post) {
                const float4 b = *reinterpret_cast<const float4*>(post + c);
                *reinterpret_cast<float4*>(h + idx) = make_float4(v[k].x + b.x, v[k].y + b.y, v[k].z + b.z, v[k].w + b.w);
            } else if (n_partials) {
                *reinterpret_cast<float4*>(h + idx) = v[k];
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (threadIdx.x + 256 * k) * 4;
        if (c < hidden) {
            const float4 g1 = *reinterpret_cast<const float4*>(gamma1 + c);
            const float nx = v[k].x * inv, ny = v[k].y * inv, nz = v[k].z * inv, nw = v[k].w * inv;
            store4(x1 + (size_t)r * hidden + c, nx * g1.x, ny * g1.y, nz * g1.z, nw * g1.w);
            if (x2) {
                const float4 g2 = *reinterpret_cast<const float4*>(gamma2 + c);
                store4(x2 + (size_t)r * hidden + c, nx * g2.x, ny * g2.y, nz * g2.z, nw * g2.w);
            }
        }
    }
}

extern "C" int idm_add_rmsnorm2(float* h, const float* delta, int n_partials, long long partial_stride,
                                const float* gamma1, const float* gamma2, float eps, void* x1, void* x2,
                                const float* post, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0, "add_rmsnorm2: bad sizes rows=%d hidden=%d", n_rows, hidden);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "add_rmsnorm2: hidden=%d does not fit shared memory", hidden);
    IDM_REQUIRE((gamma2 == nullptr) == (x2 == nullptr), "add_rmsnorm2: a second weight and a second output come together");
    if (hidden % 4 == 0 && hidden <= 4096 && (partial_stride % 4) == 0) {
        // NOTE: the sum of squares is taken over the same values in another thread layout than the general kernel's;
        // which kernel runs depends on `hidden` only
        const int np = delta ? n_partials : 0;
        if (hidden <= 1024)
            idm_launch(add_rmsnorm2_vec4_kernel<1>, dim3(n_rows), dim3(256), 0, stream, h, delta, np, (size_t)partial_stride,
                       gamma1, gamma2, eps, (T*)x1, (T*)x2, post, hidden);
        else if (hidden <= 2048)
            idm_launch(add_rmsnorm2_vec4_kernel<2>, dim3(n_rows), dim3(256), 0, stream, h, delta, np, (size_t)partial_stride,
                       gamma1, gamma2, eps, (T*)x1, (T*)x2, post, hidden);
        else
            idm_launch(add_rmsnorm2_vec4_kernel<4>, dim3(n_rows), dim3(256), 0, stream, h, delta, np, (size_t)partial_stride,
                       gamma1, gamma2, eps, (T*)x1, (T*)x2, post, hidden);
        IDM_LAUNCH_CHECK("add_rmsnorm2");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(add_rmsnorm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(add_rmsnorm2_kernel, dim3(n_rows), dim3(256), smem, stream, h, delta, delta ? n_partials : 0,
               (size_t)partial_stride, gamma1, gamma2, eps, (T*)x1, (T*)x2, post, hidden);
    IDM_LAUNCH_CHECK("add_rmsnorm2");
    return 0;
}

// ---------------------------------------------------------------- rotary table
// cs[t, j] = (cos, sin)(positions[t] * inv_freq[j]), angle and functions in 64-bit,
// rounded to 32-bit (src/detllm/ops/rope.py:25-35 builds its table the same way).
// cs_by_dim, if given, gets the same values as [half, n_tokens]: there the tokens of one dim lie side
// by side, which is how a kernel with one thread per token wants to read them.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float2* __restrict__ cs, float2* __restrict__ cs_by_dim, int n_tokens, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    const int t = i / half, j = i % half;
    double s, c;
    sincos((double)positions[t] * inv_freq[j], &s, &c);
    cs[i] = make_float2((float)c, (float)s);
    if (cs_by_dim != nullptr) cs_by_dim[(size_t)j * n_tokens + t] = make_float2((float)c, (float)s);
}

extern "C" int idm_rope_table(const int* positions, const double* inv_freq, float* cs, float* cs_by_dim,
                              int n_tokens, int half, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(half > 0, "rope_table: bad half=%d", half);
    const int n = n_tokens * half;
    idm_launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, positions, inv_freq, (float2*)cs,
               (float2*)cs_by_dim, n_tokens, half);
    IDM_LAUNCH_CHECK("rope_table");
    return 0;
}

// ------------------------------------------- q/k norm + rotation + cache write
// One warp per (token, head) over the n_q + 2 n_kv heads of the fused projection.
// q and k heads: RMS norm over head_dim with a weight of shape [head_dim] shared by
// all heads (src/detllm/model.py:208-215), then rotation of pairs (d, d + hd/2)
// by the token's position (src/detllm/ops/rope.py:47-55); v heads are copied.
// q goes to q_out [N, n_q, hd]; k and v go to the cache at the token's position
// and/or to packed buffers k_new, v_new [N, n_kv, hd].
__global__ void __launch_bounds__(128) qkv_finish_kernel(QkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    // one block per token: the token's place in the cache is looked up once, the warps share the heads
    __shared__ int place[2];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.n_q + 2 * a.n_kv;
    if (threadIdx.x == 0 && a.write_cache) {
        const int pos = a.positions[t];
        const int r = a.cache.ring ? pos % a.cache.ring : pos;
        place[0] = a.cache.table[(size_t)a.slots[a.token_seq[t]] * a.cache.table_stride + r / IDM_PAGE];
        place[1] = r % IDM_PAGE;
    }
    __syncthreads();
    const int page = place[0], prow = place[1];
    if (a.tiles4) {
        // whole heads inside tiles of 128 features, four features per lane (qkv_finish_tile4)
        const int width = heads * a.hd;
        for (int f0 = warp * 128; f0 < width; f0 += 4 * 128) {
            const int f = f0 + lane * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f < width) {
                const float* p = a.qkv + (size_t)t * width + f;
                for (int z = 0; z < a.n_partials; ++z) {
                    const float4 q4 = *reinterpret_cast<const float4*>(p + (size_t)z * a.partial_stride);
                    v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w;
                }
            }
            qkv_finish_tile4(a, v, t, f0, lane, page, prow);
        }
        return;
    }
    for (int head = warp; head < heads; head += 4) {
        const size_t row = (size_t)t * heads * a.hd + (size_t)head * a.hd;
        qkv_finish_row(a, t, head, lane,
                       [&](int j) { return add_partials(0.f, a.qkv, a.n_partials, a.partial_stride, row + j); },
                       [&](int g) { return (((size_t)page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.hd; });
    }
}

extern "C" int idm_qkv_finish(const float* qkv, int n_partials, long long partial_stride, int n_tokens,
                              int n_q, int n_kv, int hd, const float* gq, const float* gk, float eps,
                              const float* cs, void* q_out, void* k_new, void* v_new,
                              void* k_pool, void* v_pool, const int* table, int table_stride, int ring,
                              const int* token_seq, const int* positions, const int* slots,
                              cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd % 2 == 0 && hd <= IDM_MAX_HEAD_DIM,
                "qkv_finish: head_dim=%d must be even and at most %d", hd, IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_q > 0 && n_kv >= 0 && n_partials >= 1, "qkv_finish: bad head counts %d/%d", n_q, n_kv);
    QkvArgs a;
    a.qkv = qkv; a.n_partials = n_partials; a.partial_stride = (size_t)partial_stride;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd;
    a.gq = gq; a.gk = gk; a.eps = eps; a.inv_hd = 1.0f / (float)hd; a.cs = (const float2*)cs; a.cs_by_dim = nullptr;
    a.q_out = (T*)q_out; a.k_new = (T*)k_new; a.v_new = (T*)v_new;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.write_cache = k_pool != nullptr;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots;
    a.tiles4 = (128 % hd == 0 && hd >= 8 && (partial_stride % 4) == 0) ? 1 : 0;
    idm_launch(qkv_finish_kernel, dim3(n_tokens), dim3(128), 0, stream, a);
    IDM_LAUNCH_CHECK("qkv_finish");
    return 0;
}

// ------------------------------------------------------------------ ring write
// After a windowed layer's attention: the step's keys and values go into the ring.
// Only a sequence's last `ring` tokens are written (earlier ones would be overwritten
// by later ones of the same step; each ring position gets exactly one writer).
__global__ void kv_write_ring_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, KVAddr c,
                                     const int* __restrict__ token_seq, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const int* __restrict__ kv_len,
                                     int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * c.n_kv) return;
    const int t = warp / c.n_kv, g = warp % c.n_kv;
    const int s = token_seq[t], pos = positions[t];
    if (c.ring && pos < kv_len[s] - c.ring) return;
    const size_t off = kv_offset(c, slots[s], pos, g);
    const size_t src = ((size_t)t * c.n_kv + g) * c.hd;
    for (int d = lane; d < c.hd; d += 32) { c.k[off + d] = k_new[src + d]; c.v[off + d] = v_new[src + d]; }
}

extern "C" int idm_kv_write_ring(const void* k_new, const void* v_new, void* k_pool, void* v_pool,
                                 const int* table, int table_stride, int ring, const int* token_seq,
                                 const int* positions, const int* slots, const int* kv_len, int n_tokens,
                                 int n_kv, int hd, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    KVAddr c{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    const long long warps = (long long)n_tokens * n_kv;
    idm_launch(kv_write_ring_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, 
        (const T*)k_new, (const T*)v_new, c, token_seq, positions, slots, kv_len, n_tokens);
    IDM_LAUNCH_CHECK("kv_write_ring");
    return 0;
}

// ---------------------------------------------------------------------- SwiGLU
// y[t, i] = g * sigmoid(g) * u  (src/detllm/ops/di_swiglu.py:43-45; float form tests/test_ops.py:240-242).
// Plain layout: g = gu[t, i], u = gu[t, inter + i].  Tiled layout (the gate/up weight's rows in tiles
// alternating: gate row of a feature, then its up row; 64 features per 128-row tile, zero rows past
// the end): g = gu[t, 128 (i / 64) + 2 (i % 64)], u = the next column.
// grid (column blocks, tokens): no division by a runtime size per element.
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gu, int n_partials, size_t partial_stride,
                                                     T* __restrict__ y, int inter, int width, int tiled) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const size_t t = blockIdx.y;
    const int gi = tiled ? ((c >> 6) << 7) + 2 * (c & 63) : c;
    const int ui = tiled ? gi + 1 : c + inter;
    const size_t base = t * (size_t)width;
    const float g = add_partials(0.f, gu, n_partials, partial_stride, base + gi);
    const float u = add_partials(0.f, gu, n_partials, partial_stride, base + ui);
    from_f32(y[t * (size_t)inter + c], silu_mul(g, u));
}

extern "C" int idm_swiglu(const float* gu, int n_partials, long long partial_stride, void* y, int n_tokens,
                          int inter, int tiled, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(inter > 0 && n_partials >= 1, "swiglu: bad sizes");
    IDM_REQUIRE(n_tokens <= 65535 * 64, "swiglu: %d tokens in one launch", n_tokens);
    const int width = tiled ? ((inter + 63) / 64) * 128 : 2 * inter;
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        idm_launch(swiglu_kernel, dim3((inter + 255) / 256, nt), dim3(256), 0, stream,
                   gu + (size_t)t0 * width, n_partials, (size_t)partial_stride, (T*)y + (size_t)t0 * inter, inter, width,
                   tiled);
        IDM_LAUNCH_CHECK("swiglu");
    }
    return 0;
}

// ------------------------------------------------------------ scaled embedding
// h[t, :] = table[tokens[t], :] * scale, the product rounded once in 32-bit
__global__ void embed_scaled_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                    float* __restrict__ h, int hidden, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + (size_t)tokens[t] * hidden;
    float* out = h + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

extern "C" int idm_embed_scaled(const int* tokens, const void* table, float* h, int n_tokens, int hidden,
                                float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(n_tokens > 0 && hidden > 0, "embed: bad sizes n_tokens=%d hidden=%d", n_tokens, hidden);
    idm_launch(embed_scaled_kernel, dim3(n_tokens), dim3(256), 0, stream, tokens, (const T*)table, h, hidden, scale);
    IDM_LAUNCH_CHECK("embed_scaled");
    return 0;
}

// ------------------------------------------- norm behind a sublayer, and the next one before
// For layers that norm a sublayer's output before adding it:
//   h[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w_post          (32-bit, stored)
// and, in the same pass over the row, what the next sublayer reads:
//   mode 1: x[r] = h[r] / sqrt(mean(h[r]^2) + eps_pre) * w_pre;   mode 2: x[r] = h[r];   mode 0: nothing.
// One block per row, the row kept in shared memory between the passes.
__global__ void __launch_bounds__(256) post_pre_norm_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                            const float* __restrict__ w_post, float eps,
                                                            const float* __restrict__ w_pre, float eps_pre,
                                                            T* __restrict__ x, int mode, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];
    const size_t r = blockIdx.x;
    const float* yr = y + r * hidden;
    float* hr = h + r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float v = yr[c]; vals[c] = v; ss = fmaf(v, v, ss); }
    float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = hr[c] + vals[c] * inv * w_post[c];
        hr[c] = v; vals[c] = v; ss = fmaf(v, v, ss);
    }
    if (mode == 0) return;
    T* xr = x + r * hidden;
    if (mode == 2) {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) from_f32(xr[c], vals[c]);
        return;
    }
    inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps_pre);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) from_f32(xr[c], vals[c] * inv * w_pre[c]);
}

// The same for rows of at most 4 * 256 elements with hidden % 4 == 0, in two forms that give the same bits: a block
// per row (a thread owns four consecutive elements), and, for many rows, a warp per row in which lane l stands for
// the block's threads l, l + 32, ..: it sums each of those warps by the same butterfly and adds the eight totals in
// the same order.  Every product and sum is written out, so that the two forms cannot be contracted differently.
struct PostPre4 { float4 y, h; };
__device__ __forceinline__ float sumsq4(const float4& v) {
    return __fmaf_rn(v.w, v.w, __fmaf_rn(v.z, v.z, __fmaf_rn(v.y, v.y, __fmul_rn(v.x, v.x))));
}
__device__ __forceinline__ float4 post_add4(const float4& h, const float4& y, float inv, const float4& w) {
    return make_float4(__fmaf_rn(__fmul_rn(y.x, inv), w.x, h.x), __fmaf_rn(__fmul_rn(y.y, inv), w.y, h.y),
                       __fmaf_rn(__fmul_rn(y.z, inv), w.z, h.z), __fmaf_rn(__fmul_rn(y.w, inv), w.w, h.w));
}
__device__ __forceinline__ void pre_store4(T* x, const float4& h, float inv, const float4& w, int mode) {
    if (mode == 2) store4(x, h.x, h.y, h.z, h.w);
    else store4(x, __fmul_rn(__fmul_rn(h.x, inv), w.x), __fmul_rn(__fmul_rn(h.y, inv), w.y), __fmul_rn(__fmul_rn(h.z, inv), w.z),
                __fmul_rn(__fmul_rn(h.w, inv), w.w));
}

__global__ void __launch_bounds__(256) post_pre_norm_vec4_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                                 const float* __restrict__ w_post, float eps,
                                                                 const float* __restrict__ w_pre, float eps_pre,
                                                                 T* __restrict__ x, int mode, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t r = blockIdx.x;
    const int c = threadIdx.x * 4;
    const bool live = c < hidden;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 yv = live ? *reinterpret_cast<const float4*>(y + r * hidden + c) : zero;
    float4 hv = live ? *reinterpret_cast<const float4*>(h + r * hidden + c) : zero;
    float inv = 1.0f / sqrtf(block_sum(sumsq4(yv), scratch) / (float)hidden + eps);
    if (live) {
        hv = post_add4(hv, yv, inv, *reinterpret_cast<const float4*>(w_post + c));
        *reinterpret_cast<float4*>(h + r * hidden + c) = hv;
    }
    if (mode == 0) return;
    inv = mode == 1 ? 1.0f / sqrtf(block_sum(sumsq4(hv), scratch) / (float)hidden + eps_pre) : 0.f;
    if (live) pre_store4(x + r * hidden + c, hv, inv, mode == 1 ? *reinterpret_cast<const float4*>(w_pre + c) : zero, mode);
}

__global__ void __launch_bounds__(256) post_pre_norm_rows_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                                 const float* __restrict__ w_post, float eps,
                                                                 const float* __restrict__ w_pre, float eps_pre,
                                                                 T* __restrict__ x, int mode, int n_rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const size_t r = i;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 yv[8], hv[8];
    float s[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        yv[w] = c < hidden ? *reinterpret_cast<const float4*>(y + r * hidden + c) : zero;
        hv[w] = c < hidden ? *reinterpret_cast<const float4*>(h + r * hidden + c) : zero;
        s[w] = sumsq4(yv[w]);
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) s[w] = warp_sum(s[w]);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += s[w];
    float inv = 1.0f / sqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        if (c < hidden) {
            hv[w] = post_add4(hv[w], yv[w], inv, *reinterpret_cast<const float4*>(w_post + c));
            *reinterpret_cast<float4*>(h + r * hidden + c) = hv[w];
        }
        s[w] = sumsq4(hv[w]);
    }
    if (mode == 0) return;
    if (mode == 1) {
#pragma unroll
        for (int w = 0; w < 8; ++w) s[w] = warp_sum(s[w]);
        total = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += s[w];
        inv = 1.0f / sqrtf(total / (float)hidden + eps_pre);
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        if (c < hidden) pre_store4(x + r * hidden + c, hv[w], inv, mode == 1 ? *reinterpret_cast<const float4*>(w_pre + c) : zero, mode);
    }
}

extern "C" int idm_post_pre_norm(float* h, const float* y, const float* w_post, float eps, const float* w_pre,
                                 float eps_pre, void* x, int mode, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0 && mode >= 0 && mode <= 2, "post_pre_norm: rows=%d hidden=%d mode=%d", n_rows, hidden, mode);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "post_pre_norm: hidden=%d does not fit shared memory", hidden);
    IDM_REQUIRE(mode == 0 || x != nullptr, "post_pre_norm: mode %d needs an output", mode);
    IDM_REQUIRE(mode != 1 || w_pre != nullptr, "post_pre_norm: mode 1 needs the next norm's weight");
    if (hidden % 4 == 0 && hidden <= 1024) {
        // which of the two runs depends on the number of rows; they give the same bits
        if (n_rows >= 64)
            idm_launch(post_pre_norm_rows_kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, h, y, w_post, eps, w_pre, eps_pre,
                       (T*)x, mode, n_rows, hidden);
        else
            idm_launch(post_pre_norm_vec4_kernel, dim3(n_rows), dim3(256), 0, stream, h, y, w_post, eps, w_pre, eps_pre, (T*)x,
                       mode, hidden);
        IDM_LAUNCH_CHECK("post_pre_norm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(post_pre_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(post_pre_norm_kernel, dim3(n_rows), dim3(256), smem, stream, h, y, w_post, eps, w_pre, eps_pre, (T*)x, mode, hidden);
    IDM_LAUNCH_CHECK("post_pre_norm");
    return 0;
}

// ------------------------------------------------------ gated activations, by name
// (gated_act in common.cuh: act 0 is g * sigmoid(g) * u, act 1 the tanh form of gelu times u)

// y[t, i] = act(gu[t, i]) * gu[t, inter + i] of a 32-bit gate/up product [N, 2 * inter]
__global__ void __launch_bounds__(256) gated_act_kernel(const float* __restrict__ gu, T* __restrict__ y, int inter, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const size_t t = blockIdx.x;
    from_f32(y[t * (size_t)inter + c], gated_act(gu[t * 2 * (size_t)inter + c], gu[t * 2 * (size_t)inter + inter + c], act));
}

extern "C" int idm_gated_act(const float* gu, void* y, int n_tokens, int inter, int act, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(inter > 0 && act >= 0 && act <= 2, "gated_act: inter=%d act=%d", inter, act);
    idm_launch(gated_act_kernel, dim3(n_tokens, (inter + 255) / 256), dim3(256), 0, stream, gu, (T*)y, inter, act);
    IDM_LAUNCH_CHECK("gated_act");
    return 0;
}

// y[t, j] = act(s[t, j]) * table[tokens[t], col0 + j]: a projection gated by a slice of the token's own row
// of a second embedding table [vocab, table_width]
__global__ void __launch_bounds__(256) token_gate_kernel(const float* __restrict__ s, const int* __restrict__ tokens,
                                                         const T* __restrict__ table, int table_width, int col0,
                                                         T* __restrict__ y, int dim, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= dim) return;
    const size_t t = blockIdx.x;
    const float e = to_f32(table[(size_t)tokens[t] * table_width + col0 + j]);
    from_f32(y[t * (size_t)dim + j], gated_act(s[t * (size_t)dim + j], e, act));
}

extern "C" int idm_token_gate(const float* s, const int* tokens, const void* table, int table_width, int col0,
                              void* y, int n_tokens, int dim, int act, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(dim > 0 && col0 >= 0 && col0 + dim <= table_width && (act == 0 || act == 1),
                "token_gate: columns %d..%d of rows of %d, act=%d", col0, col0 + dim, table_width, act);
    idm_launch(token_gate_kernel, dim3(n_tokens, (dim + 255) / 256), dim3(256), 0, stream, s, tokens, (const T*)table,
               table_width, col0, (T*)y, dim, act);
    IDM_LAUNCH_CHECK("token_gate");
    return 0;
}

// ------------------------------------------------------------- output gate of a mixer
// out[t, out_col + c] = o[t, c] * sigmoid(gate[t * gate_stride + c]) * scale   (gate null: only the constant);
// o [N, width] in the storage type, gate 32-bit (columns of a wider projection), out rows of out_stride.
__global__ void __launch_bounds__(256) gate_scale_kernel(const T* __restrict__ o, const float* __restrict__ gate,
                                                         int gate_stride, int gate_group, float scale, T* __restrict__ out,
                                                         int out_stride, int out_col, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= width) return;
    const size_t t = blockIdx.x;
    const T* src = o + t * width + c;
    T* dst = out + t * out_stride + out_col + c;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (c + i >= width) break;
        float v = to_f32(src[i]);
        if (gate) v = v / (1.0f + expf(-gate[t * gate_stride + (c + i) / gate_group]));
        from_f32(dst[i], v * scale);
    }
}

extern "C" int idm_gate_scale(const void* o, const float* gate, int gate_stride, int gate_group, float scale, void* out,
                              int out_stride, int out_col, int n_tokens, int width, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(width > 0 && out_col >= 0 && out_col + width <= out_stride, "gate_scale: columns %d..%d of rows of %d", out_col,
                out_col + width, out_stride);
    IDM_REQUIRE(gate_group >= 1, "gate_scale: a gate serves %d columns", gate_group);
    idm_launch(gate_scale_kernel, dim3(n_tokens, (width + 1023) / 1024), dim3(256), 0, stream, (const T*)o, gate, gate_stride,
               gate_group, scale, (T*)out, out_stride, out_col, width);
    IDM_LAUNCH_CHECK("gate_scale");
    return 0;
}

// ------------------------------------------------------- residual add + a norm without statistics
// The same interface as add_rmsnorm (rows == nullptr: h[r] += sum_p delta[p][r], stored, x[r] = f(h[r]); rows given:
// only those rows, nothing stored) with f(v) = tanh(alpha v) * w + b, element by element, in 32-bit.
__global__ void __launch_bounds__(256) add_dyt_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                      size_t partial_stride, const float* __restrict__ w,
                                                      const float* __restrict__ b, float alpha, T* __restrict__ x,
                                                      const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * hidden;
    T* xr = x + (size_t)i * hidden;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hidden; c += gridDim.y * blockDim.x) {
        const float v = add_partials(hr[c], delta, n_partials, partial_stride, (size_t)r * hidden + c);
        if (!rows && n_partials) hr[c] = v;
        from_f32(xr[c], fmaf(tanhf(alpha * v), w[c], b[c]));
    }
}

extern "C" int idm_add_dyt(float* h, const float* delta, int n_partials, long long partial_stride, const float* w,
                           const float* b, float alpha, void* x, const int* rows, int n_rows, int hidden,
                           cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0, "add_dyt: bad sizes rows=%d hidden=%d", n_rows, hidden);
    // few rows: a row's elements over several blocks (nothing is summed over a row, so the split changes no value)
    const int by = n_rows >= 128 ? 1 : max(1, min((hidden + 255) / 256, 128 / n_rows));
    idm_launch(add_dyt_kernel, dim3(n_rows, by), dim3(256), 0, stream, h, delta, delta ? n_partials : 0, (size_t)partial_stride,
               w, b, alpha, (T*)x, rows, hidden);
    IDM_LAUNCH_CHECK("add_dyt");
    return 0;
}

// ------------------------------------------------------- an activation of one argument, 32-bit in, storage type out
// act 2: relu(z)^2
__global__ void __launch_bounds__(256) act_cast_kernel(const float* __restrict__ z, T* __restrict__ y, size_t n, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = fmaxf(z[i], 0.f);
    from_f32(y[i], v * v);
}

// four elements per thread (n % 4 == 0): the same values
__global__ void __launch_bounds__(256) act_cast4_kernel(const float* __restrict__ z, T* __restrict__ y, size_t n4, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 v = *reinterpret_cast<const float4*>(z + 4 * i);
    const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
    store4(y + 4 * i, a * a, b * b, c * c, d * d);
}

extern "C" int idm_act_cast(const float* z, void* y, long long n, int act, cudaStream_t stream) {
    if (n == 0) return 0;
    IDM_REQUIRE(act == 2, "act_cast: activation %d is not built (2: the square of relu)", act);
    if (n % 4 == 0 && ((uintptr_t)z % 16) == 0 && ((uintptr_t)y % 16) == 0)
        idm_launch(act_cast4_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, z, (T*)y, (size_t)(n / 4), act);
    else
        idm_launch(act_cast_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, z, (T*)y, (size_t)n, act);
    IDM_LAUNCH_CHECK("act_cast");
    return 0;
}

// ------------------------------------------------------- the stream and a second stream side by side
// h[r] += sum_p delta[p][r] (stored), out[r] = [h[r] | x0[r]] in the storage type: the input of a product that
// mixes the running stream with an earlier one.
__global__ void __launch_bounds__(256) concat_cast_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                          size_t partial_stride, const float* __restrict__ x0,
                                                          T* __restrict__ out, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = add_partials(h[r * hidden + c], delta, n_partials, partial_stride, r * hidden + c);
        if (n_partials) h[r * hidden + c] = v;
        from_f32(out[r * 2 * hidden + c], v);
        from_f32(out[r * 2 * hidden + hidden + c], x0[r * hidden + c]);
    }
}

extern "C" int idm_concat_cast(float* h, const float* delta, int n_partials, long long partial_stride, const float* x0,
                               void* out, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    idm_launch(concat_cast_kernel, dim3(n_rows), dim3(256), 0, stream, h, delta, delta ? n_partials : 0, (size_t)partial_stride, x0,
               (T*)out, hidden);
    IDM_LAUNCH_CHECK("concat_cast");
    return 0;
}

// ------------------------------------------------------- logits times a constant, then a soft cap
// l <- cap * tanh(l * scale / cap)  (cap <= 0: l * scale alone), in place
__global__ void __launch_bounds__(256) logit_cap_kernel(float* __restrict__ l, size_t n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = l[i] * scale;
    l[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

extern "C" int idm_logit_cap(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    idm_launch(logit_cap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, logits, (size_t)n, scale, cap);
    IDM_LAUNCH_CHECK("logit_cap");
    return 0;
}

#if defined(IDM_BF16)
// h += down . act(up . x) from one call: the up product (32-bit z), the activation (y, storage type), the down
// product added into the stream: the calls a dense feed-forward makes, with the same arguments
extern "C" int idm_gemm_bf16(const void* x, const void* w, float* out, int M, int N, int K, cudaStream_t stream);
extern "C" int idm_gemm_bf16_residual(const void* x, const void* w, float* h, int M, int N, int K, cudaStream_t stream);

extern "C" int idm_dense_ff(const void* x, const void* w_up, const void* w_down, float* z, void* y, float* h, int n_tokens,
                            int width, int ff, int act, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    if (idm_gemm_bf16(x, w_up, z, n_tokens, ff, width, stream)) return 1;
    if (idm_act_cast(z, y, (long long)n_tokens * ff, act, stream)) return 1;
    return idm_gemm_bf16_residual(y, w_down, h, n_tokens, width, ff, stream);
}
#endif
