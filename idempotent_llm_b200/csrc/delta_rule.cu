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
// With one decay per head (head_col >= 0) the projection is proj[t, head_col + h], dt_bias has H entries, and the
// head's decay is written to all dk of its columns of `a`, which the recurrence reads as it reads decays per channel.
struct DeltaPrepArgs {
    float* c; int c_stride, c_q, c_k;
    float* a; int a_stride, a_col;
    const float* proj; int p_stride, b_col, head_col;
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
        const int hh = i / p.dk;
        const float rate = expf(p.a_log[hh]);
        const float z = p.head_col >= 0 ? p.proj[(size_t)t * p.p_stride + p.head_col + hh] + p.dt_bias[hh] : arow[i] + p.dt_bias[i];
        arow[i] = expf(-rate * softplus_f(z));
    }
    for (int h = blockIdx.y * blockDim.x + threadIdx.x; h < p.H; h += gridDim.y * blockDim.x)
        p.beta[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-p.proj[(size_t)t * p.p_stride + p.b_col + h]));
}

extern "C" int idm_delta_prep(float* c, int c_stride, int c_q, int c_k, float* a, int a_stride, int a_col,
                              const float* proj, int p_stride, int b_col, int head_col, const float* dt_bias, const float* a_log,
                              float* beta, int H, int Hk, int dk, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && Hk > 0 && H % Hk == 0 && dk > 0, "delta_prep: %d heads over %d key heads of %d", H, Hk, dk);
    DeltaPrepArgs p{c, c_stride, c_q, c_k, a, a_stride, a_col, proj, p_stride, b_col, head_col, dt_bias, a_log, beta, H, Hk, dk};
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
    const bool vec = a.dk % 4 == 0 && ((uintptr_t)sp & 15) == 0;      // a thread's rows as 16-byte pieces
#pragma unroll
    for (int i = 0; i < RP; i += 4) {
        if (vec) {
            const float4 x = (col && row0 + i < a.dk) ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
        } else {
#pragma unroll
            for (int e = i; e < i + 4; ++e) S[e] = (col && row0 + e < a.dk) ? sp[e] : 0.f;
        }
    }

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
        for (int i = 0; i < RP; i += 4) {
            if (vec) {
                if (row0 + i < a.dk) *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
            } else {
#pragma unroll
                for (int e = i; e < i + 4; ++e)
                    if (row0 + e < a.dk) sp[e] = S[e];
            }
        }
    }
}

// The same recurrence for portions of many tokens.  Walking a portion token by token from global memory pays a
// load's latency per token; here a block brings DS_TOK tokens' q, k, g, its 16 columns of v and beta into shared
// memory with asynchronous copies, two stages deep, and the walk reads them from there.  Element d = r RP + i of a
// head's q, k or g lies at ((i / 4) 8 + r) 4 + i % 4 of its row, so that the eight threads of a column read 128
// bytes side by side.  The arithmetic and its order are those of the kernel above: both give the same bits.
__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int RP>
struct DeltaStage {
    static constexpr int DKP = RP * 8;                          // a head's key size, rounded up to the threads' rows
    static constexpr int TOK = RP <= 16 ? 16 : 8;               // tokens per stage
    static constexpr int ROW = 3 * DKP + DS_COLS + 4;           // k, q, g, v of the block's columns, beta (and 3 unused)
    static constexpr int FLOATS = 2 * TOK * ROW;
};

template <int RP, bool VEC>
__global__ void __launch_bounds__(DS_COLS * 8) delta_scan_staged_kernel(DeltaScanArgs a) {
    using St = DeltaStage<RP>;
    extern __shared__ __align__(16) float ds_smem[];
    pdl_launch_dependents();
    const int s = blockIdx.z, h = blockIdx.y, hk = h / (a.H / a.Hk);
    const int tid = threadIdx.x, r = tid & 7, jl = tid >> 3, j0 = blockIdx.x * DS_COLS, j = j0 + jl;
    const bool col = j < a.dv;
    const int row0 = r * RP;
    // rows past dk are never copied: k = q = 0 and g = 1 there, once for both stages
    for (int e = tid; e < 2 * St::TOK * St::DKP; e += DS_COLS * 8) {
        const int row = e / St::DKP, p = e % St::DKP;
        const int d = (p >> 2 & 7) * RP + (p >> 5) * 4 + (p & 3);
        if (d >= a.dk) {
            float* base = ds_smem + row * St::ROW;
            base[p] = 0.f; base[St::DKP + p] = 0.f; base[2 * St::DKP + p] = 1.f;
        }
    }
    pdl_wait();
    const int t0 = a.cu_q[s], t1 = a.cu_q[s + 1];
    float* sp = a.state + (size_t)a.slots[s] * a.state_stride + ((size_t)h * a.dv + (col ? j : 0)) * a.dk + row0;
    float S[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) S[i] = (col && row0 + i < a.dk) ? sp[i] : 0.f;

    const int cols = min(DS_COLS, a.dv - j0);
    auto issue = [&](int tb, int stage) {
        const int n = min(St::TOK, t1 - tb);
        float* st = ds_smem + stage * St::TOK * St::ROW;
        if (VEC) {
            const int per = a.dk >> 2, total = n * 3 * per;
            for (int e = tid; e < total; e += DS_COLS * 8) {
                const int tt = e / (3 * per), w = e % (3 * per), which = w / per, d = (w % per) << 2;
                const float* src = which == 2 ? a.g + (size_t)(tb + tt) * a.g_stride + a.g_col + h * a.dk + d
                                              : a.c + (size_t)(tb + tt) * a.c_stride + (which ? a.c_q : a.c_k) + hk * a.dk + d;
                const int rr = d / RP, i = d % RP;
                cp_async_16(st + tt * St::ROW + which * St::DKP + (((i >> 2) * 8 + rr) << 2), src);
            }
        } else {
            const int total = n * 3 * a.dk;
            for (int e = tid; e < total; e += DS_COLS * 8) {
                const int tt = e / (3 * a.dk), w = e % (3 * a.dk), which = w / a.dk, d = w % a.dk;
                const float* src = which == 2 ? a.g + (size_t)(tb + tt) * a.g_stride + a.g_col + h * a.dk + d
                                              : a.c + (size_t)(tb + tt) * a.c_stride + (which ? a.c_q : a.c_k) + hk * a.dk + d;
                const int rr = d / RP, i = d % RP;
                cp_async_4(st + tt * St::ROW + which * St::DKP + (((i >> 2) * 8 + rr) << 2) + (i & 3), src);
            }
        }
        for (int e = tid; e < n * (cols + 1); e += DS_COLS * 8) {
            const int tt = e / (cols + 1), c = e % (cols + 1);
            const float* src = c < cols ? a.c + (size_t)(tb + tt) * a.c_stride + a.c_v + h * a.dv + j0 + c
                                        : a.beta + (size_t)(tb + tt) * a.H + h;
            cp_async_4(st + tt * St::ROW + 3 * St::DKP + (c < cols ? c : DS_COLS), src);
        }
        cp_async_commit();
    };

    const int n_chunks = (t1 - t0 + St::TOK - 1) / St::TOK;
    if (n_chunks > 0) issue(t0, 0);
    for (int ch = 0; ch < n_chunks; ++ch) {
        const int tb = t0 + ch * St::TOK;
        if (ch + 1 < n_chunks) { issue(tb + St::TOK, (ch + 1) & 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const float* st = ds_smem + (ch & 1) * St::TOK * St::ROW;
        const int n = min(St::TOK, t1 - tb);
        for (int tt = 0; tt < n; ++tt) {
            const float* row = st + tt * St::ROW;
            const float v = row[3 * St::DKP + jl], beta = row[3 * St::DKP + DS_COLS];
            float kr[RP];
            float sk = 0.f, sq = 0.f, kk = 0.f;
#pragma unroll
            for (int m = 0; m < RP / 4; ++m) {
                const float4 k4 = *reinterpret_cast<const float4*>(row + ((m * 8 + r) << 2));
                const float4 q4 = *reinterpret_cast<const float4*>(row + St::DKP + ((m * 8 + r) << 2));
                const float4 g4 = *reinterpret_cast<const float4*>(row + 2 * St::DKP + ((m * 8 + r) << 2));
                const float kx[4] = {k4.x, k4.y, k4.z, k4.w}, qx[4] = {q4.x, q4.y, q4.z, q4.w}, gx[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float& Sv = S[m * 4 + i];
                    Sv *= gx[i];
                    sk = fmaf(Sv, kx[i], sk);
                    sq = fmaf(Sv, qx[i], sq);
                    kk = fmaf(kx[i], qx[i], kk);
                    kr[m * 4 + i] = kx[i];
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
                kk += __shfl_xor_sync(0xffffffffu, kk, o);
            }
            const float u = beta * (v - sk);
#pragma unroll
            for (int i = 0; i < RP; ++i) S[i] = fmaf(kr[i], u, S[i]);
            if (col && r == 0) a.o[(size_t)(tb + tt) * a.o_stride + h * a.dv + j] = fmaf(u, kk, sq);
        }
        __syncthreads();
    }
    if (col) {
#pragma unroll
        for (int i = 0; i < RP; ++i)
            if (row0 + i < a.dk) sp[i] = S[i];
    }
}

template <int RP>
static int delta_scan_staged(const DeltaScanArgs& a, dim3 grid, cudaStream_t stream) {
    const size_t smem = (size_t)DeltaStage<RP>::FLOATS * sizeof(float);
    const bool vec = a.dk % 4 == 0 && a.c_stride % 4 == 0 && a.c_q % 4 == 0 && a.c_k % 4 == 0 && a.g_stride % 4 == 0 &&
                     a.g_col % 4 == 0 && ((uintptr_t)a.c & 15) == 0 && ((uintptr_t)a.g & 15) == 0;
    static bool set[2] = {false, false};
    if (!set[vec]) {
        cudaError_t e = vec ? cudaFuncSetAttribute(delta_scan_staged_kernel<RP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(delta_scan_staged_kernel<RP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        IDM_REQUIRE(e == cudaSuccess, "delta_scan: %zu bytes of shared memory were refused (%s)", smem, cudaGetErrorString(e));
        set[vec] = true;
    }
    if (vec) idm_launch(delta_scan_staged_kernel<RP, true>, grid, dim3(DS_COLS * 8), smem, stream, a);
    else idm_launch(delta_scan_staged_kernel<RP, false>, grid, dim3(DS_COLS * 8), smem, stream, a);
    return 0;
}

// ------------------------------------------------------------------ the recurrence, sixteen tokens at a time
// Over a chunk of C tokens that starts from the state S0, with G_t the product of the decays up to and including
// token t (per key channel), the walk above unrolls to
//
//   u_t  = beta_t (v_t - S0^T (G_t k_t) - sum_{s<t} A_ts u_s),      A_ts = sum_d k_s[d] k_t[d] G_t[d] / G_s[d]
//   o_t  = S0^T (G_t q_t) + sum_{s<=t} B_ts u_s,                    B_ts = sum_d k_s[d] q_t[d] G_t[d] / G_s[d]
//   S_C  = G_C S0 + sum_s (k_s G_C / G_s) u_s^T
//
// so that the work against the state becomes three products with C independent sums each instead of a chain of
// C dependent steps, and the chain that is left (the u_t, a triangular system of C unknowns per column) is C short
// steps in registers.  The quotients G_t / G_s are never divided out: they are products of the decays between s
// and t, in (0, 1], so a decay that underflows ends at 0 and nothing overflows.  A and B belong to (chunk, head)
// and not to a column: a pass of its own makes them for all chunks side by side.  All of it is 32-bit; the numbers
// are those of the walk up to the order of the sums.
#define DC_C 16                                                 // tokens per chunk

// ab[(t H + h) 2C ..]: for token s of a chunk, -A_ts for the chunk's tokens t > s (0 elsewhere), then B_ts for t >= s
__global__ void __launch_bounds__(128) delta_pairs_kernel(DeltaScanArgs a, float* __restrict__ ab) {
    __shared__ float sm[3][DC_C][128];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.z, h = blockIdx.y, hk = h / (a.H / a.Hk), tid = threadIdx.x;
    const int t0 = a.cu_q[s], t1 = a.cu_q[s + 1], tb = t0 + blockIdx.x * DC_C;
    if (tb >= t1) return;
    const int n = min(DC_C, t1 - tb);
    for (int e = tid; e < n * a.dk; e += 128) {
        const int tt = e / a.dk, d = e % a.dk;
        const float* row = a.c + (size_t)(tb + tt) * a.c_stride + hk * a.dk + d;
        sm[0][tt][d] = row[a.c_k];
        sm[1][tt][d] = row[a.c_q];
        sm[2][tt][d] = a.g[(size_t)(tb + tt) * a.g_stride + a.g_col + h * a.dk + d];
    }
    for (int e = tid; e < n * 2 * DC_C; e += 128)
        ab[((size_t)(tb + e / (2 * DC_C)) * a.H + h) * (2 * DC_C) + e % (2 * DC_C)] = 0.f;
    __syncthreads();
    // a warp takes four tokens s whose rows together are as long as every other warp's; its lanes split the channels
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
        const int ts = pass == 0 ? warp : pass == 1 ? 7 - warp : pass == 2 ? 8 + warp : 15 - warp;
        if (ts >= n) continue;
        float kr[4];                                            // k_s times the decays from s up to the token at hand
#pragma unroll
        for (int i = 0; i < 4; ++i) kr[i] = lane + 32 * i < a.dk ? sm[0][ts][lane + 32 * i] : 0.f;
        float* out = ab + ((size_t)(tb + ts) * a.H + h) * (2 * DC_C);
        for (int t = ts; t < n; ++t) {
            float pa = 0.f, pb = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dk) {
                    if (t > ts) kr[i] *= sm[2][t][d];
                    pa = fmaf(sm[0][t][d], kr[i], pa);
                    pb = fmaf(sm[1][t][d], kr[i], pb);
                }
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                pa += __shfl_xor_sync(0xffffffffu, pa, o);
                pb += __shfl_xor_sync(0xffffffffu, pb, o);
            }
            if (lane == 0) {
                if (t > ts) out[t] = -pa;
                out[DC_C + t] = pb;
            }
        }
    }
}

// The chunk kernel: a block owns (sequence, head, 16 columns of S), a warp four of the columns, lane L rows
// [L RP, (L + 1) RP) of each.  Four columns a warp, because what a warp reads from shared memory (a token's scaled k or
// q) then serves four sums, and four independent chains keep one warp per scheduler busy.  Per chunk: (1) the threads
// turn the staged k, q, g in place into k G_C / G_t, q G_t, k G_t, a thread per channel and group of tokens, the
// groups' products joined through shared memory; (2) the warp lays its columns of S0 into shared memory, and lane t
// sums S0^T (G_t k_t) for token t's correction, lane 16 + t S0^T (G_t q_t) for its read-out; (3) the triangular system
// runs down the lanes: u_s goes from lane s to all, lane L adds row s's entry L of [-A | B] times u_s to its sum; (4)
// lanes 16.. store the read-outs, all lanes bring their rows of S behind the chunk.
#define DC_NC 4                                                 // columns per warp
template <int RP>
struct DeltaChunk {
    static constexpr int DKP = RP * 32, NT = DS_COLS / DC_NC * 32;
    static constexpr int NG = NT / DKP < 1 ? 1 : NT / DKP;      // groups of tokens in step (1)
    static constexpr int V_AT = 3 * DKP, BETA_AT = V_AT + DS_COLS, AB_AT = BETA_AT + 4;
    static constexpr int ROW = AB_AT + 2 * DC_C;                // k, q, g, v of the block's columns, beta, -A and B
    static constexpr int GC_AT = 2 * DC_C * ROW;                // the chunk's whole decay, behind the two stages
    static constexpr int GP_AT = GC_AT + DKP;                   // the token groups' decays
    static constexpr int SW_AT = GP_AT + NG * DKP;              // the block's columns of S
    static constexpr int FLOATS = SW_AT + DS_COLS * DKP;
    static_assert(DKP <= NT && DC_C % NG == 0, "a thread per channel, whole groups of tokens");
};

template <int RP>
__device__ __forceinline__ void load_rows(const float* p, float (&x)[RP]) {
    if constexpr (RP == 4) { const float4 v = *reinterpret_cast<const float4*>(p); x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w; }
    else if constexpr (RP == 2) { const float2 v = *reinterpret_cast<const float2*>(p); x[0] = v.x; x[1] = v.y; }
    else x[0] = *p;
}

template <int RP, bool VEC>
__global__ void __launch_bounds__(DeltaChunk<RP>::NT) delta_scan_chunked_kernel(DeltaScanArgs a, const float* __restrict__ ab) {
    using L = DeltaChunk<RP>;
    constexpr int C = DC_C, NT = L::NT, NC = DC_NC, NW = NT / 32;
    extern __shared__ __align__(16) float ds_smem[];
    pdl_launch_dependents();
    const int s = blockIdx.z, h = blockIdx.y, hk = h / (a.H / a.Hk);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, j0 = blockIdx.x * DS_COLS, jw = warp * NC;
    const int row0 = lane * RP;
    for (int e = tid; e < 2 * C * L::DKP; e += NT) {            // channels past dk: k = q = 0, g = 1, never copied
        const int row = e / L::DKP, p = e % L::DKP;
        if (p >= a.dk) {
            float* base = ds_smem + row * L::ROW;
            base[p] = 0.f; base[L::DKP + p] = 0.f; base[2 * L::DKP + p] = 1.f;
        }
    }
    pdl_wait();
    const int t0 = a.cu_q[s], t1 = a.cu_q[s + 1];
    float* sp = a.state + (size_t)a.slots[s] * a.state_stride + ((size_t)h * a.dv + j0 + jw) * a.dk + row0;
    float S[NC][RP];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < RP; ++i) S[c][i] = (j0 + jw + c < a.dv && row0 + i < a.dk) ? sp[(size_t)c * a.dk + i] : 0.f;

    const int cols = min(DS_COLS, a.dv - j0);
    auto issue = [&](int tb, int stage) {
        const int n = min(C, t1 - tb);
        for (int tt = warp; tt < n; tt += NW) {
            const int t = tb + tt;
            float* row = ds_smem + (stage * C + tt) * L::ROW;
            const float* kp = a.c + (size_t)t * a.c_stride + hk * a.dk;
            const float* gp = a.g + (size_t)t * a.g_stride + a.g_col + h * a.dk;
            if (VEC) {
                for (int d = lane * 4; d < a.dk; d += 128) {
                    cp_async_16(row + d, kp + a.c_k + d);
                    cp_async_16(row + L::DKP + d, kp + a.c_q + d);
                    cp_async_16(row + 2 * L::DKP + d, gp + d);
                }
            } else {
                for (int d = lane; d < a.dk; d += 32) {
                    cp_async_4(row + d, kp + a.c_k + d);
                    cp_async_4(row + L::DKP + d, kp + a.c_q + d);
                    cp_async_4(row + 2 * L::DKP + d, gp + d);
                }
            }
            if (lane < cols) cp_async_4(row + L::V_AT + lane, a.c + (size_t)t * a.c_stride + a.c_v + h * a.dv + j0 + lane);
            else if (lane == 16) cp_async_4(row + L::BETA_AT, a.beta + (size_t)t * a.H + h);
            else if (lane >= 24) cp_async_16(row + L::AB_AT + (lane - 24) * 4, ab + ((size_t)t * a.H + h) * (2 * C) + (lane - 24) * 4);
        }
        cp_async_commit();
    };

    const int n_chunks = (t1 - t0 + C - 1) / C;
    if (n_chunks > 0) issue(t0, 0);
    for (int ch = 0; ch < n_chunks; ++ch) {
        const int tb = t0 + ch * C;
        if (ch + 1 < n_chunks) { issue(tb + C, (ch + 1) & 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        float* st = ds_smem + (ch & 1) * C * L::ROW;
        const int n = min(C, t1 - tb);
        // a last chunk of fewer tokens: the missing ones write nothing (k = 0, beta = 0) and decay nothing (g = 1)
        for (int e = tid; e < (C - n) * L::ROW; e += NT) {
            const int c = e % L::ROW;
            st[(n + e / L::ROW) * L::ROW + c] = (c >= 2 * L::DKP && c < 3 * L::DKP) ? 1.f : 0.f;
        }
        __syncthreads();
        // (1) in place, per channel: k -> k G_C / G_t, q -> q G_t, g -> k G_t; and G_C.  Thread (channel, group of tokens).
        {
            constexpr int TPG = C / L::NG;
            const int p = tid % L::DKP, grp = tid / L::DKP;
            float gg[TPG], kk[TPG], qq[TPG];
            if (grp < L::NG) {
                float prod = 1.f;
#pragma unroll
                for (int i = 0; i < TPG; ++i) {
                    const float* row = st + (TPG * grp + i) * L::ROW;
                    gg[i] = row[2 * L::DKP + p]; kk[i] = row[p]; qq[i] = row[L::DKP + p];
                    prod *= gg[i];
                }
                if (L::NG > 1) ds_smem[L::GP_AT + grp * L::DKP + p] = prod;
            }
            if (L::NG > 1) __syncthreads();
            if (grp < L::NG) {
                float G = 1.f, suf = 1.f;
                if (L::NG > 1) {
#pragma unroll
                    for (int o = 0; o < L::NG; ++o) {
                        const float x = ds_smem[L::GP_AT + o * L::DKP + p];
                        if (o < grp) G *= x;
                        if (o > grp) suf *= x;
                    }
                }
#pragma unroll
                for (int i = 0; i < TPG; ++i) {
                    float* row = st + (TPG * grp + i) * L::ROW;
                    G *= gg[i];
                    row[2 * L::DKP + p] = kk[i] * G;
                    row[L::DKP + p] = qq[i] * G;
                }
                if (grp == L::NG - 1) ds_smem[L::GC_AT + p] = G;
#pragma unroll
                for (int i = TPG - 1; i >= 0; --i) {
                    st[(TPG * grp + i) * L::ROW + p] = kk[i] * suf;
                    suf *= gg[i];
                }
            }
        }
        __syncthreads();
        // (2) what the state before the chunk gives token t's correction (lane t) and read-out (lane 16 + t): the columns
        // go through shared memory, and a lane walks all of them against its token's G_t k_t or G_t q_t
        float x[NC];
        {
            float* sw = ds_smem + L::SW_AT + jw * L::DKP;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                if constexpr (RP == 4) *reinterpret_cast<float4*>(sw + c * L::DKP + row0) = make_float4(S[c][0], S[c][1], S[c][2], S[c][3]);
                else if constexpr (RP == 2) *reinterpret_cast<float2*>(sw + c * L::DKP + row0) = make_float2(S[c][0], S[c][1]);
                else sw[c * L::DKP + row0] = S[c][0];
            }
            __syncwarp();
            const float* xr = st + (lane & 15) * L::ROW + (lane < 16 ? 2 * L::DKP : L::DKP);
            float acc[NC][4];
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
#pragma unroll 8
            for (int m = 0; m < L::DKP / 4; ++m) {
                const float4 xv = *reinterpret_cast<const float4*>(xr + 4 * m);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const float4 sv = *reinterpret_cast<const float4*>(sw + c * L::DKP + 4 * m);
                    acc[c][0] = fmaf(xv.x, sv.x, acc[c][0]); acc[c][1] = fmaf(xv.y, sv.y, acc[c][1]);
                    acc[c][2] = fmaf(xv.z, sv.z, acc[c][2]); acc[c][3] = fmaf(xv.w, sv.w, acc[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) x[c] = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
        }
        // (3) lane t < 16: v_t minus the sum, times beta_t when its turn comes; lane 16 + t: the read-out so far
        float u[NC][C];
        const float* mine = st + (lane & 15) * L::ROW;
        const float beta = lane < 16 ? mine[L::BETA_AT] : 0.f;
        if (lane < 16) {
#pragma unroll
            for (int c = 0; c < NC; ++c) x[c] = (j0 + jw + c < a.dv ? mine[L::V_AT + jw + c] : 0.f) - x[c];
        }
#pragma unroll
        for (int q = 0; q < C; ++q) {
            const float coef = st[q * L::ROW + L::AB_AT + lane];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                u[c][q] = __shfl_sync(0xffffffffu, beta * x[c], q);
                x[c] = fmaf(coef, u[c][q], x[c]);
            }
        }
        if (lane >= 16 && lane - 16 < n) {
            float* dst = a.o + (size_t)(tb + lane - 16) * a.o_stride + h * a.dv + j0 + jw;
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (j0 + jw + c < a.dv) dst[c] = x[c];
        }
        // (4) the state behind the chunk
        {
            float gc[RP];
            load_rows<RP>(ds_smem + L::GC_AT + row0, gc);
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int i = 0; i < RP; ++i) S[c][i] *= gc[i];
        }
#pragma unroll
        for (int t = 0; t < C; ++t) {
            float kt[RP];
            load_rows<RP>(st + t * L::ROW + row0, kt);
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
                for (int i = 0; i < RP; ++i) S[c][i] = fmaf(kt[i], u[c][t], S[c][i]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < RP; ++i)
            if (j0 + jw + c < a.dv && row0 + i < a.dk) sp[(size_t)c * a.dk + i] = S[c][i];
}

template <int RP>
static int delta_scan_chunked(const DeltaScanArgs& a, float* ab, dim3 grid, int max_tokens, cudaStream_t stream) {
    const size_t smem = (size_t)DeltaChunk<RP>::FLOATS * sizeof(float);
    const bool vec = a.dk % 4 == 0 && a.c_stride % 4 == 0 && a.c_q % 4 == 0 && a.c_k % 4 == 0 && a.g_stride % 4 == 0 &&
                     a.g_col % 4 == 0 && ((uintptr_t)a.c & 15) == 0 && ((uintptr_t)a.g & 15) == 0;
    static bool set[2] = {false, false};
    if (!set[vec]) {
        cudaError_t e = vec ? cudaFuncSetAttribute(delta_scan_chunked_kernel<RP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(delta_scan_chunked_kernel<RP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        IDM_REQUIRE(e == cudaSuccess, "delta_scan: %zu bytes of shared memory were refused (%s)", smem, cudaGetErrorString(e));
        set[vec] = true;
    }
    idm_launch(delta_pairs_kernel, dim3((max_tokens + DC_C - 1) / DC_C, grid.y, grid.z), dim3(128), 0, stream, a, ab);
    if (vec) idm_launch(delta_scan_chunked_kernel<RP, true>, grid, dim3(DeltaChunk<RP>::NT), smem, stream, a, (const float*)ab);
    else idm_launch(delta_scan_chunked_kernel<RP, false>, grid, dim3(DeltaChunk<RP>::NT), smem, stream, a, (const float*)ab);
    return 0;
}

// Floats of scratch that a step of `n_tokens` tokens, at most `max_tokens` of one sequence, wants (0: none).
extern "C" long long idm_delta_scan_scratch_floats(int n_tokens, int H, int dk, int max_tokens) {
    return (max_tokens > 4 && dk <= 128) ? (long long)n_tokens * H * 2 * DC_C : 0;
}

// `max_tokens`: the most tokens any sequence brings to this step; steps of a few tokens walk them straight from
// global memory, longer portions run in chunks (keys of at most 128, with `scratch` of
// idm_delta_scan_scratch_floats) or walk through shared memory.
extern "C" int idm_delta_scan(const float* c, int c_stride, int c_q, int c_k, int c_v, const float* g, int g_stride,
                              int g_col, const float* beta, float* state, long long state_stride, float* o,
                              int o_stride, const int* cu_q, const int* slots, int n_seqs, int H, int Hk, int dk,
                              int dv, int max_tokens, float* scratch, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    IDM_REQUIRE(H > 0 && Hk > 0 && H % Hk == 0 && dk > 0 && dk <= 256 && dv > 0, "delta_scan: %d heads over %d key heads, "
                "keys of %d (at most 256), values of %d", H, Hk, dk, dv);
    IDM_REQUIRE(state != nullptr && state_stride >= (long long)H * dk * dv, "delta_scan: a slot's state must hold %d x %d x %d floats",
                H, dv, dk);
    IDM_REQUIRE(n_seqs <= 65535 && H <= 65535, "delta_scan: %d sequences, %d heads in one launch", n_seqs, H);
    DeltaScanArgs a{c, c_stride, c_q, c_k, c_v, g, g_stride, g_col, beta, state, state_stride, o, o_stride, cu_q, slots,
                    H, Hk, dk, dv};
    const dim3 grid((dv + DS_COLS - 1) / DS_COLS, H, n_seqs), block(DS_COLS * 8);
    if (max_tokens > 4 && dk <= 128 && scratch != nullptr) {
        IDM_REQUIRE(((uintptr_t)scratch & 15) == 0 && (max_tokens + DC_C - 1) / DC_C <= 0x7fffffff, "delta_scan: scratch at %p", (void*)scratch);
        int rc;
        if (dk <= 32) rc = delta_scan_chunked<1>(a, scratch, grid, max_tokens, stream);
        else if (dk <= 64) rc = delta_scan_chunked<2>(a, scratch, grid, max_tokens, stream);
        else rc = delta_scan_chunked<4>(a, scratch, grid, max_tokens, stream);
        if (rc) return rc;
    } else if (max_tokens > 4) {
        int rc;
        if (dk <= 32) rc = delta_scan_staged<4>(a, grid, stream);
        else if (dk <= 64) rc = delta_scan_staged<8>(a, grid, stream);
        else if (dk <= 128) rc = delta_scan_staged<16>(a, grid, stream);
        else rc = delta_scan_staged<32>(a, grid, stream);
        if (rc) return rc;
    } else if (dk <= 32) idm_launch(delta_scan_kernel<4>, grid, block, 0, stream, a);
    else if (dk <= 64) idm_launch(delta_scan_kernel<8>, grid, block, 0, stream, a);
    else if (dk <= 128) idm_launch(delta_scan_kernel<16>, grid, block, 0, stream, a);
    else idm_launch(delta_scan_kernel<32>, grid, block, 0, stream, a);
    IDM_LAUNCH_CHECK("delta_scan");
    return 0;
}

// ------------------------------------------------------------------ behind the recurrence
// out[t, out_col + h dv + j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * w[j] * act(gate[t, gate_col + h dv + j]) * scale,
// act = sigmoid (gate_act 0) or silu (gate_act 1); one warp per (token, head)
__global__ void __launch_bounds__(128) delta_out_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ w,
                                                        float eps, const float* __restrict__ gate, int gate_stride,
                                                        int gate_col, int gate_act, float scale, T* __restrict__ out,
                                                        int out_stride, int out_col, int n_tokens, int H, int dv) {
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
    for (int d = lane; d < dv; d += 32) {
        const float z = gr[d], sg = 1.0f / (1.0f + expf(-z));
        from_f32(dst[d], gate_act == 1 ? x[d] * inv * w[d] * (z * sg) * scale : x[d] * inv * w[d] / (1.0f + expf(-z)) * scale);
    }
}

extern "C" int idm_delta_out(const float* o, int o_stride, const float* w, float eps, const float* gate, int gate_stride,
                             int gate_col, int gate_act, float scale, void* out, int out_stride, int out_col, int n_tokens, int H,
                             int dv, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(H > 0 && dv > 0 && out_col >= 0 && out_col + H * dv <= out_stride, "delta_out: columns %d..%d of rows of %d",
                out_col, out_col + H * dv, out_stride);
    const long long warps = (long long)n_tokens * H;
    idm_launch(delta_out_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, o, o_stride, w, eps, gate,
               gate_stride, gate_col, gate_act, scale, (T*)out, out_stride, out_col, n_tokens, H, dv);
    IDM_LAUNCH_CHECK("delta_out");
    return 0;
}
