// The gated delta rule: a recurrent mixer whose state S [dk, dv] per head is decayed row by row, corrected
// towards the token's value at the token's key, and read with the token's query:
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// q, k [Hk, dk] are unit vectors per head (q also times dk^-1/2), v [H, dv], beta [H] in (0, 1), g [H, dk] in (0, 1];
// head h reads q/k head h / (H / Hk).  Everything here is 32-bit: the state, the decays and their logarithms, the
// unit norms, the gates.  S lives per sequence as [H][dv][dk] (a column's dk numbers side by side) and is carried
// from step to step; tokens are walked one by one from and to it, so a token's result does not depend on how its
// sequence was cut into steps.
//
// The read-out is computed from the decayed state before the write: o = (g S)^T q + u (k . q), the same number
// as S_new^T q, so that one round of shuffles per token serves both sums.
#include "common.cuh"

// ------------------------------------------------------------------ columns of a 32-bit buffer as a matrix operand
// out[t, c] = in[t, col0 + c] for c < width, 0 for width <= c < out_width, in the storage type
__global__ void __launch_bounds__(256) cols_cast_kernel(const float* __restrict__ in, int stride, int col0, int width,
                                                        T* __restrict__ out, int out_width, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n * out_width) return;
    const int t = (int)(i / out_width), c = (int)(i % out_width);
    from_f32(out[i], c < width ? in[(size_t)t * stride + col0 + c] : 0.f);
}

extern "C" int idm_cols_cast(const float* in, int stride, int col0, int width, void* out, int out_width, int n_tokens,
                             cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(col0 >= 0 && width > 0 && col0 + width <= stride && out_width >= width,
                "cols_cast: columns %d..%d of rows of %d into rows of %d", col0, col0 + width, stride, out_width);
    const long long total = (long long)n_tokens * out_width;
    idm_launch(cols_cast_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, in, stride, col0, width,
               (T*)out, out_width, n_tokens);
    IDM_LAUNCH_CHECK("cols_cast");
    return 0;
}

// ------------------------------------------------------------------ what the recurrence reads, made in place
// c [N, c_stride]: filtered and activated q (Hk x dk at c_q), k (at c_k); both become unit vectors per head,
// x / sqrt(sum x^2 + 1e-6), q also times dk^-1/2.  a [N, a_stride]: columns [a_col, a_col + H dk) hold the decay's
// projection and become g = exp(-exp(A_log[h]) * softplus(a + dt_bias)).  beta[t, h] = sigmoid(proj[t, b_col + h]).
struct DeltaPrepArgs {
    float* c; int c_stride, c_q, c_k;
    float* a; int a_stride, a_col;
    const float* proj; int p_stride, b_col;
    const float* dt_bias; const float* a_log;
    float* beta;
    int H, Hk, dk;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__global__ void __launch_bounds__(128) delta_prep_kernel(DeltaPrepArgs p) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* row = p.c + (size_t)t * p.c_stride;
    const float q_scale = 1.0f / sqrtf((float)p.dk);
    for (int i = blockIdx.y * 4 + warp; i < 2 * p.Hk; i += gridDim.y * 4) {
        const bool is_q = i < p.Hk;
        float* x = row + (is_q ? p.c_q + i * p.dk : p.c_k + (i - p.Hk) * p.dk);
        float ss = 0.f;
        for (int d = lane; d < p.dk; d += 32) ss += x[d] * x[d];
        const float inv = (is_q ? q_scale : 1.f) / sqrtf(warp_sum(ss) + 1e-6f);
        for (int d = lane; d < p.dk; d += 32) x[d] *= inv;
    }
    float* arow = p.a + (size_t)t * p.a_stride + p.a_col;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < p.H * p.dk; i += gridDim.y * blockDim.x) {
        const float rate = expf(p.a_log[i / p.dk]);
        arow[i] = expf(-rate * softplus_f(arow[i] + p.dt_bias[i]));
    }
    for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < p.H; h += gridDim.y * blockDim.x)
        p.beta[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-p.proj[(size_t)t * p.p_stride + p.b_col + h]));
}

extern "C" int idm_delta_prep(float* c, int c_stride, int c_q, int c_k, float* a, int a_stride, int a_col,
                              const float* proj, int p_stride, int b_col, const float* dt_bias, const float* a_log,
                              float* beta, int H, int Hk, int dk, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && Hk > 0 && H % Hk == 0 && dk > 0, "delta_prep: %d heads over %d key heads of %d", H, Hk, dk);
    DeltaPrepArgs p{c, c_stride, c_q, c_k, a, a_stride, a_col, proj, p_stride, b_col, dt_bias, a_log, beta, H, Hk, dk};
    int split = (296 + n_tokens - 1) / n_tokens;
    const int most = (H * dk + 127) / 128;
    if (split > most) split = most;
    if (split < 1) split = 1;
    idm_launch(delta_prep_kernel, dim3(n_tokens, split), dim3(128), 0, stream, p);
    IDM_LAUNCH_CHECK("delta_prep");
    return 0;
}

// ------------------------------------------------------------------ the recurrence
// A block owns (sequence, head, 16 columns of S).  Eight threads share a column: thread r of them keeps rows
// [r RP, (r + 1) RP) of it in registers, and the eight add their parts of a column's sums by three shuffles.  The
// next token's q, k, g are loaded while this token's sums are on their way.
struct DeltaScanArgs {
    const float* c; int c_stride, c_q, c_k, c_v;      // q, k unit vectors [Hk, dk]; v [H, dv]
    const float* g; int g_stride, g_col;              // decays [H, dk]
    const float* beta;                                // [N, H]
    float* state; long long state_stride;             // state + slot * state_stride : [H][dv][dk]
    float* o; int o_stride;                           // o[t, h * dv + j]
    const int* cu_q; const int* slots;
    int H, Hk, dk, dv;
};

#define DS_COLS 16

template <int RP>
__global__ void __launch_bounds__(DS_COLS * 8) delta_scan_kernel(DeltaScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.z, h = blockIdx.y, hk = h / (a.H / a.Hk);
    const int r = threadIdx.x & 7, j = blockIdx.x * DS_COLS + (threadIdx.x >> 3);
    const bool col = j < a.dv;
    const int row0 = r * RP;
    const int t0 = a.cu_q[s], t1 = a.cu_q[s + 1];
    float* sp = a.state + (size_t)a.slots[s] * a.state_stride + ((size_t)h * a.dv + (col ? j : 0)) * a.dk + row0;
    float S[RP], kq[3][RP];                           // (k, q, g of the token at hand)
#pragma unroll
    for (int i = 0; i < RP; ++i) S[i] = (col && row0 + i < a.dk) ? sp[i] : 0.f;

    auto load = [&](int t, float (&dst)[3][RP]) {
        const float* kp = a.c + (size_t)t * a.c_stride + a.c_k + hk * a.dk + row0;
        const float* qp = a.c + (size_t)t * a.c_stride + a.c_q + hk * a.dk + row0;
        const float* gp = a.g + (size_t)t * a.g_stride + a.g_col + h * a.dk + row0;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            const bool live = row0 + i < a.dk;
            dst[0][i] = live ? kp[i] : 0.f;
            dst[1][i] = live ? qp[i] : 0.f;
            dst[2][i] = live ? gp[i] : 1.f;
        }
    };
    if (t0 < t1) load(t0, kq);
    for (int t = t0; t < t1; ++t) {
        float nx[3][RP];
        if (t + 1 < t1) load(t + 1, nx);
        const float v = col ? a.c[(size_t)t * a.c_stride + a.c_v + h * a.dv + j] : 0.f;
        const float beta = a.beta[(size_t)t * a.H + h];
        float sk = 0.f, sq = 0.f, kk = 0.f;
#pragma unroll
        for (int i = 0; i < RP; ++i) {
            S[i] *= kq[2][i];
            sk = fmaf(S[i], kq[0][i], sk);
            sq = fmaf(S[i], kq[1][i], sq);
            kk = fmaf(kq[0][i], kq[1][i], kk);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            kk += __shfl_xor_sync(0xffffffffu, kk, o);
        }
        const float u = beta * (v - sk);
#pragma unroll
        for (int i = 0; i < RP; ++i) S[i] = fmaf(kq[0][i], u, S[i]);
        if (col && r == 0) a.o[(size_t)t * a.o_stride + h * a.dv + j] = fmaf(u, kk, sq);
        if (t + 1 < t1) {
#pragma unroll
            for (int i = 0; i < RP; ++i) { kq[0][i] = nx[0][i]; kq[1][i] = nx[1][i]; kq[2][i] = nx[2][i]; }
        }
    }
    if (col) {
#pragma unroll
        for (int i = 0; i < RP; ++i)
            if (row0 + i < a.dk) sp[i] = S[i];
    }
}

extern "C" int idm_delta_scan(const float* c, int c_stride, int c_q, int c_k, int c_v, const float* g, int g_stride,
                              int g_col, const float* beta, float* state, long long state_stride, float* o,
                              int o_stride, const int* cu_q, const int* slots, int n_seqs, int H, int Hk, int dk,
                              int dv, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    IDM_REQUIRE(H > 0 && Hk > 0 && H % Hk == 0 && dk > 0 && dk <= 256 && dv > 0, "delta_scan: %d heads over %d key heads, "
                "keys of %d (at most 256), values of %d", H, Hk, dk, dv);
    IDM_REQUIRE(state != nullptr && state_stride >= (long long)H * dk * dv, "delta_scan: a slot's state must hold %d x %d x %d floats",
                H, dv, dk);
    IDM_REQUIRE(n_seqs <= 65535 && H <= 65535, "delta_scan: %d sequences, %d heads in one launch", n_seqs, H);
    DeltaScanArgs a{c, c_stride, c_q, c_k, c_v, g, g_stride, g_col, beta, state, state_stride, o, o_stride, cu_q, slots,
                    H, Hk, dk, dv};
    const dim3 grid((dv + DS_COLS - 1) / DS_COLS, H, n_seqs), block(DS_COLS * 8);
    if (dk <= 32) idm_launch(delta_scan_kernel<4>, grid, block, 0, stream, a);
    else if (dk <= 64) idm_launch(delta_scan_kernel<8>, grid, block, 0, stream, a);
    else if (dk <= 128) idm_launch(delta_scan_kernel<16>, grid, block, 0, stream, a);
    else idm_launch(delta_scan_kernel<32>, grid, block, 0, stream, a);
    IDM_LAUNCH_CHECK("delta_scan");
    return 0;
}

// ------------------------------------------------------------------ behind the recurrence
// out[t, out_col + h dv + j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * w[j] * sigmoid(gate[t, gate_col + h dv + j]) * scale,
// one warp per (token, head)
__global__ void __launch_bounds__(128) delta_out_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ w,
                                                        float eps, const float* __restrict__ gate, int gate_stride,
                                                        int gate_col, float scale, T* __restrict__ out, int out_stride,
                                                        int out_col, int n_tokens, int H, int dv) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= (long long)n_tokens * H) return;
    const int t = (int)(i / H), h = (int)(i % H);
    const float* x = o + (size_t)t * o_stride + (size_t)h * dv;
    float ss = 0.f;
    for (int d = lane; d < dv; d += 32) ss += x[d] * x[d];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    const float* gr = gate + (size_t)t * gate_stride + gate_col + (size_t)h * dv;
    T* dst = out + (size_t)t * out_stride + out_col + (size_t)h * dv;
    for (int d = lane; d < dv; d += 32)
        from_f32(dst[d], x[d] * inv * w[d] / (1.0f + expf(-gr[d])) * scale);
}

extern "C" int idm_delta_out(const float* o, int o_stride, const float* w, float eps, const float* gate, int gate_stride,
                             int gate_col, float scale, void* out, int out_stride, int out_col, int n_tokens, int H,
                             int dv, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && dv > 0 && out_col >= 0 && out_col + H * dv <= out_stride, "delta_out: columns %d..%d of rows of %d",
                out_col, out_col + H * dv, out_stride);
    const long long warps = (long long)n_tokens * H;
    idm_launch(delta_out_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, o, o_stride, w, eps, gate,
               gate_stride, gate_col, scale, (T*)out, out_stride, out_col, n_tokens, H, dv);
    IDM_LAUNCH_CHECK("delta_out");
    return 0;
}
