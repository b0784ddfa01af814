// What lies between a joint q/k/v projection and an attention over the cache, for mixers whose projections have
// biases, whose q and k heads are normed, whose rotation covers part of a head, and whose values may be the keys
// themselves as projected:
//
//   q_h = turn(norm(W_q x + b_q)_h)      k_g = turn(norm(W_k x + b_k)_g)      v_g = (W_v x + b_v)_g   or   (W_k x + b_k)_g
//
// norm: x / sqrt(mean(x^2) + eps) * weight over a head, one weight [dk] for all heads (absent: no norm);
// turn: the first 2 * half dims of a head, dim i with dim i + half, (u, v) -> (u c - v s, v c + u s) with (c, s) =
// mag * (cos, sin) of the token's row of the table (half 0: no rotation).  Everything in 32-bit; q is stored
// [N, n_q, dk] in the storage type, k and v go to the token's place in the cache.  One warp per (token, head).
#include "common.cuh"

struct HeadFinishArgs {
    const float* proj; int stride;            // the step's projections [N, stride], 32-bit
    int col_q, col_k, col_v;                  // first columns of q, k and v heads; col_v < 0: values are the keys as projected
    const float* bias_q; const float* bias_k; const float* bias_v;     // [heads * size] or null
    const float* gamma_q; const float* gamma_k;                        // [dk] or null
    float eps;
    int half; const float2* cs; float mag;    // table [N, half] of (cos, sin)
    int n_q, n_kv, dk, dv;
    T* q_out;
    KVAddr cache;                             // k rows of dk, v rows of dv
    const int* token_seq; const int* positions; const int* slots;
};

#define HF_WARPS 4
#define HF_PER_LANE (IDM_MAX_HEAD_DIM / 32)

__global__ void __launch_bounds__(HF_WARPS * 32) head_finish_kernel(HeadFinishArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];           // a head per warp, for the rotation's partner dims
    __shared__ int place[2];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        const int pos = a.positions[t];
        const int r = a.cache.ring ? pos % a.cache.ring : pos;
        place[0] = a.cache.table[(size_t)a.slots[a.token_seq[t]] * a.cache.table_stride + r / IDM_PAGE];
        place[1] = r % IDM_PAGE;
    }
    __syncthreads();
    const size_t page = place[0], prow = place[1];
    float* mine = smem + warp * a.dk;
    const float* row = a.proj + (size_t)t * a.stride;
    const int own_v = a.col_v >= 0 ? a.n_kv : 0;
    for (int head = blockIdx.y * HF_WARPS + warp; head < a.n_q + a.n_kv + own_v; head += gridDim.y * HF_WARPS) {
        if (head >= a.n_q + a.n_kv) {         // a value head of its own: bias, cast, store
            const int g = head - a.n_q - a.n_kv;
            T* dst = a.cache.v + ((page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.dv;
            for (int d = lane; d < a.dv; d += 32) {
                float v = row[a.col_v + g * a.dv + d];
                if (a.bias_v) v += a.bias_v[g * a.dv + d];
                from_f32(dst[d], v);
            }
            continue;
        }
        const bool is_q = head < a.n_q;
        const int g = is_q ? head : head - a.n_q;
        const float* src = row + (is_q ? a.col_q : a.col_k) + g * a.dk;
        const float* bias = is_q ? a.bias_q : a.bias_k;
        const float* gamma = is_q ? a.gamma_q : a.gamma_k;
        float x[HF_PER_LANE];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < HF_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            x[i] = 0.f;
            if (d < a.dk) {
                x[i] = src[d] + (bias ? bias[g * a.dk + d] : 0.f);
                ss += x[i] * x[i];
            }
        }
        if (!is_q && a.col_v < 0) {           // the key as projected is the value
            T* dst = a.cache.v + ((page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.dv;
#pragma unroll
            for (int i = 0; i < HF_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dk) from_f32(dst[d], x[i]);
            }
        }
        if (gamma) {
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.dk + a.eps);
#pragma unroll
            for (int i = 0; i < HF_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dk) x[i] = x[i] * inv * gamma[d];
            }
        }
        T* dst = is_q ? a.q_out + ((size_t)t * a.n_q + g) * a.dk
                      : a.cache.k + ((page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.dk;
        if (a.half) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < HF_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dk) mine[d] = x[i];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < HF_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < 2 * a.half) {
                    const int j = d < a.half ? d : d - a.half;
                    const float2 cs = a.cs[(size_t)t * a.half + j];
                    const float c = cs.x * a.mag, s = cs.y * a.mag;
                    const float other = mine[d < a.half ? d + a.half : d - a.half];
                    x[i] = d < a.half ? x[i] * c - other * s : x[i] * c + other * s;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < HF_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < a.dk) from_f32(dst[d], x[i]);
        }
    }
}

extern "C" int idm_head_finish(const float* proj, int stride, int col_q, int col_k, int col_v, const float* bias_q,
                               const float* bias_k, const float* bias_v, const float* gamma_q, const float* gamma_k,
                               float eps, int half, const float* cs, float mag, int n_q, int n_kv, int dk, int dv,
                               void* q_out, void* k_pool, void* v_pool, const int* table, int table_stride, int ring,
                               const int* token_seq, const int* positions, const int* slots, int n_tokens,
                               cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(n_q > 0 && n_kv > 0 && dk > 0 && dk <= IDM_MAX_HEAD_DIM && dv > 0 && dv <= IDM_MAX_HEAD_DIM,
                "head_finish: heads %d/%d of sizes %d/%d (at most %d)", n_q, n_kv, dk, dv, IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(half >= 0 && 2 * half <= dk && (half == 0 || cs != nullptr), "head_finish: %d turning pairs in heads of %d", half, dk);
    IDM_REQUIRE(col_v >= 0 || dv == dk, "head_finish: keys of %d cannot be values of %d", dk, dv);
    const int last = col_v >= 0 ? col_v + n_kv * dv : 0;
    IDM_REQUIRE(col_q >= 0 && col_k >= 0 && col_q + n_q * dk <= stride && col_k + n_kv * dk <= stride && last <= stride,
                "head_finish: columns beyond rows of %d", stride);
    HeadFinishArgs a;
    a.proj = proj; a.stride = stride; a.col_q = col_q; a.col_k = col_k; a.col_v = col_v;
    a.bias_q = bias_q; a.bias_k = bias_k; a.bias_v = bias_v; a.gamma_q = gamma_q; a.gamma_k = gamma_k; a.eps = eps;
    a.half = half; a.cs = (const float2*)cs; a.mag = mag; a.n_q = n_q; a.n_kv = n_kv; a.dk = dk; a.dv = dv;
    a.q_out = (T*)q_out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, dk};
    a.token_seq = token_seq; a.positions = positions; a.slots = slots;
    // a block of four warps per token; steps of few tokens spread a token's heads over several blocks
    const int heads = n_q + n_kv + (col_v >= 0 ? n_kv : 0);
    int split = (296 + n_tokens - 1) / n_tokens;
    if (split > (heads + HF_WARPS - 1) / HF_WARPS) split = (heads + HF_WARPS - 1) / HF_WARPS;
    if (split < 1) split = 1;
    idm_launch(head_finish_kernel, dim3(n_tokens, split), dim3(HF_WARPS * 32), HF_WARPS * dk * sizeof(float), stream, a);
    IDM_LAUNCH_CHECK("head_finish");
    return 0;
}
