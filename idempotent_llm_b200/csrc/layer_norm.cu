// Layer norm with weight and bias, in the two places a decoder has it, and the token embedding with a hashed
// bigram row added.
//
//   LN(v) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w + b          all in 32-bit
//
// The mean is taken first and the squared deviations from it second (two passes over a row that is kept on chip),
// so that rows whose mean is large against their spread lose nothing.  Sums run in a fixed order that depends on the
// row's length only: a row's result does not depend on how many rows the step holds.
#include "common.cuh"

// ------------------------------------------------------- the norm BEHIND a sublayer, with a learned scale
// For layers that norm a sublayer's output, scale it row-wise and add it to the stream (the sublayers read the
// stream itself, there is no norm in front of them):
//   h[r] += scale * LN(y[r])            stored, 32-bit;  scale: [hidden] or null
//   mode 2: x[r] = h[r] in the storage type (what the next sublayer's products read);  mode 0: nothing.
// One block per row, the row in shared memory between the passes.
__global__ void __launch_bounds__(256) post_layernorm_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                             const float* __restrict__ w, const float* __restrict__ b,
                                                             const float* __restrict__ scale, float eps,
                                                             T* __restrict__ x, int mode, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];
    const size_t r = blockIdx.x;
    const float* yr = y + r * hidden;
    float* hr = h + r * hidden;
    float s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float v = yr[c]; vals[c] = v; s += v; }
    const float mean = block_sum(s, scratch) / (float)hidden;
    s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float d = vals[c] - mean; s = fmaf(d, d, s); }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    T* xr = mode == 2 ? x + r * hidden : nullptr;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float n = fmaf((vals[c] - mean) * inv, w[c], b[c]);
        if (scale) n *= scale[c];
        const float v = hr[c] + n;
        hr[c] = v;
        if (xr) from_f32(xr[c], v);
    }
}

// Rows of at most 1024 elements with hidden % 4 == 0: a warp per row, a lane owns up to eight groups of four
// consecutive elements, no block-wide barrier.  Blocks of eight rows when the step has many, of one row when it has
// few: the arithmetic of a row is the same.
__global__ void __launch_bounds__(256) post_layernorm_rows_kernel(float* __restrict__ h, const float* __restrict__ y,
                                                                  const float* __restrict__ w, const float* __restrict__ b,
                                                                  const float* __restrict__ scale, float eps,
                                                                  T* __restrict__ x, int mode, int n_rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const size_t r = i;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 yv[8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int c = (32 * k + lane) * 4;
        yv[k] = c < hidden ? *reinterpret_cast<const float4*>(y + r * hidden + c) : zero;
        s += (yv[k].x + yv[k].y) + (yv[k].z + yv[k].w);
    }
    const float mean = warp_sum(s) / (float)hidden;
    s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int c = (32 * k + lane) * 4;
        if (c < hidden) {
            yv[k].x -= mean; yv[k].y -= mean; yv[k].z -= mean; yv[k].w -= mean;
            s = fmaf(yv[k].x, yv[k].x, s); s = fmaf(yv[k].y, yv[k].y, s); s = fmaf(yv[k].z, yv[k].z, s); s = fmaf(yv[k].w, yv[k].w, s);
        }
    }
    const float inv = 1.0f / sqrtf(warp_sum(s) / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int c = (32 * k + lane) * 4;
        if (c < hidden) {
            const float4 wv = *reinterpret_cast<const float4*>(w + c), bv = *reinterpret_cast<const float4*>(b + c);
            float4 n = make_float4(fmaf(yv[k].x * inv, wv.x, bv.x), fmaf(yv[k].y * inv, wv.y, bv.y),
                                   fmaf(yv[k].z * inv, wv.z, bv.z), fmaf(yv[k].w * inv, wv.w, bv.w));
            if (scale) {
                const float4 sv = *reinterpret_cast<const float4*>(scale + c);
                n.x *= sv.x; n.y *= sv.y; n.z *= sv.z; n.w *= sv.w;
            }
            float4 hv = *reinterpret_cast<const float4*>(h + r * hidden + c);
            hv.x += n.x; hv.y += n.y; hv.z += n.z; hv.w += n.w;
            *reinterpret_cast<float4*>(h + r * hidden + c) = hv;
            if (mode == 2) store4(x + r * hidden + c, hv.x, hv.y, hv.z, hv.w);
        }
    }
}

extern "C" int idm_post_layernorm(float* h, const float* y, const float* w, const float* b, const float* scale, float eps,
                                  void* x, int mode, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0 && (mode == 0 || mode == 2), "post_layernorm: rows=%d hidden=%d mode=%d", n_rows, hidden, mode);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "post_layernorm: hidden=%d does not fit shared memory", hidden);
    IDM_REQUIRE(mode == 0 || x != nullptr, "post_layernorm: mode %d needs an output", mode);
    if (hidden % 4 == 0 && hidden <= 1024) {
        const int per = n_rows >= 64 ? 8 : 1;
        idm_launch(post_layernorm_rows_kernel, dim3((n_rows + per - 1) / per), dim3(32 * per), 0, stream, h, y, w, b, scale, eps, (T*)x,
                   mode, n_rows, hidden);
        IDM_LAUNCH_CHECK("post_layernorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(post_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(post_layernorm_kernel, dim3(n_rows), dim3(256), smem, stream, h, y, w, b, scale, eps, (T*)x, mode, hidden);
    IDM_LAUNCH_CHECK("post_layernorm");
    return 0;
}

// ------------------------------------------------------- residual add + layer norm (a norm in front, or the last one)
// rows == nullptr: for every row r: h[r] += sum_p delta[p][r] (stored), x[r] = LN(h[r]).
// rows != nullptr: for i < n_rows: v = h[rows[i]] + sum_p delta[p][rows[i]] (not stored), x[i] = LN(v).
__global__ void __launch_bounds__(256) add_layernorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                                            size_t partial_stride, const float* __restrict__ w,
                                                            const float* __restrict__ b, float eps, T* __restrict__ x,
                                                            const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * hidden;
    float s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = add_partials(hr[c], delta, n_partials, partial_stride, (size_t)r * hidden + c);
        if (!rows && n_partials) hr[c] = v;
        vals[c] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    s = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) { const float d = vals[c] - mean; s = fmaf(d, d, s); }
    const float inv = 1.0f / sqrtf(block_sum(s, scratch) / (float)hidden + eps);
    T* xr = x + (size_t)i * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) from_f32(xr[c], fmaf((vals[c] - mean) * inv, w[c], b[c]));
}

extern "C" int idm_add_layernorm(float* h, const float* delta, int n_partials, long long partial_stride, const float* w,
                                 const float* b, float eps, void* x, const int* rows, int n_rows, int hidden,
                                 cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0, "add_layernorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "add_layernorm: hidden=%d does not fit shared memory", hidden);
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(add_layernorm_kernel, dim3(n_rows), dim3(256), smem, stream, h, delta, delta ? n_partials : 0, (size_t)partial_stride,
               w, b, eps, (T*)x, rows, hidden);
    IDM_LAUNCH_CHECK("add_layernorm");
    return 0;
}

// ------------------------------------------------------- embedding plus a hashed bigram row
// h[t] = table[token_t] + bigram[row_t];  row_t = (prev_t * mul_prev + token_t * mul_cur) mod buckets, and row `buckets`
// (the table's last) for a sequence's first token.  prev_t is the token before t in its sequence: the step's own
// token before it, or, for the first token a sequence brings to this step, the sequence's last token of the step
// before, which lives in `last[slot * last_stride]`.  The thread block of a sequence's first token of the step reads
// that number and then writes the sequence's last token of THIS step there: nobody else touches it.  x (or null)
// receives the row in the storage type, which is what a first sublayer without a norm in front of it reads.
__global__ void __launch_bounds__(256) embed_bigram_kernel(const int* __restrict__ tokens, const int* __restrict__ token_seq,
                                                           const int* __restrict__ positions, const int* __restrict__ cu_q,
                                                           const int* __restrict__ slots, const T* __restrict__ table,
                                                           const T* __restrict__ bigram, int* __restrict__ last,
                                                           long long last_stride, float* __restrict__ h, T* __restrict__ x,
                                                           int hidden, long long buckets, long long mul_prev, long long mul_cur) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ long long row_s;
    const int t = blockIdx.x;
    if (threadIdx.x == 0) {
        const int s = token_seq[t], first = cu_q[s], tok = tokens[t];
        long long prev = -1;
        if (t > first) prev = tokens[t - 1];
        else {
            int* mine = last + (size_t)slots[s] * last_stride;
            if (positions[t] > 0) prev = *mine;
            *mine = tokens[cu_q[s + 1] - 1];
        }
        // (a product of two numbers below 2^31 fits 64 bits; the sum of two such products too)
        row_s = prev < 0 ? buckets : (prev * mul_prev + (long long)tok * mul_cur) % buckets;
    }
    __syncthreads();
    const T* erow = table + (size_t)tokens[t] * hidden;
    const T* brow = bigram + (size_t)row_s * hidden;
    float* out = h + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32(erow[i]) + to_f32(brow[i]);
        out[i] = v;
        if (x) from_f32(x[(size_t)t * hidden + i], v);
    }
}

extern "C" int idm_embed_bigram(const int* tokens, const int* token_seq, const int* positions, const int* cu_q, const int* slots,
                                const void* table, const void* bigram, int* last, long long last_stride, float* h, void* x,
                                int n_tokens, int hidden, long long buckets, long long mul_prev, long long mul_cur,
                                cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hidden > 0 && buckets > 0 && mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1LL << 31) && mul_cur < (1LL << 31),
                "embed_bigram: hidden=%d buckets=%lld factors %lld, %lld", hidden, buckets, mul_prev, mul_cur);
    IDM_REQUIRE(last != nullptr && last_stride > 0, "embed_bigram: every sequence needs a place for its last token");
    idm_launch(embed_bigram_kernel, dim3(n_tokens), dim3(256), 0, stream, tokens, token_seq, positions, cu_q, slots, (const T*)table,
               (const T*)bigram, last, last_stride, h, (T*)x, hidden, buckets, mul_prev, mul_cur);
    IDM_LAUNCH_CHECK("embed_bigram");
    return 0;
}
