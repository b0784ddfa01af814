// Attention over the cache for any head size (multiple of 8 up to 256), any number of
// heads and groups, with or without a window, for prompts and for single tokens:
// one warp per (token, q-head), all arithmetic in 32-bit.
//
// A query at position p of sequence s sees keys j with max(0, p - window + 1) <= j <= p
// (window <= 0: all j <= p), the slot-causal rule of src/detllm/model.py:259-266; with keep_first > 0 also the
// keys j < keep_first, however far back they lie (the blocks of 32 that hold them are walked first, then the
// window's).  softcap > 0 bounds a score: cap * tanh(score / cap), after the scale and before the softmax.
// Keys are walked in blocks of 32 aligned to absolute positions; inside a block lane i
// scores key j0 + i; masked lanes contribute exactly 0 and are left out of the maximum
// (the float analogue of the reference's integer sentinel, src/detllm/ops/di_softmax.py:45-58);
// the running (max, sum, context) is rescaled block by block.  The order of every sum
// depends on the query's position only, never on the step's batch or on how the
// sequence was cut into steps.
//
// Keys of the current step may come from packed buffers k_new/v_new instead of the
// cache (windowed layers, whose ring cannot hold a whole prompt).
#include "common.cuh"

struct AttnArgs {
    const T* q; T* out;
    KVAddr cache;
    const T* k_new; const T* v_new;
    const int* token_seq; const int* positions; const int* slots; const int* q_start; const int* cu_q;
    int n_tokens, n_q, n_kv, hd;
    float scale; int window;
    // beyond plain attention (all off in idm_attention_generic):
    int dv;                       // width of a value row (keys have hd)
    const float* sink;            // [n_q] or null: exp(sink[head]) joins the softmax's denominator, with no key and no value
    const float* gate; int gate_stride;   // or null: out *= sigmoid(gate[t * gate_stride + head * dv + d])
    int out_stride, out_col;      // out[t * out_stride + out_col + head * dv + d]
    float out_scale;
    const float* slopes;          // [n_q] or null: slopes[head] * (p - j) is taken off the score of key j
    int gate_per_head;            // the gate is one number per head: gate[t * gate_stride + head]
    float softcap;                // > 0: score <- softcap * tanh(score / softcap)
    int keep_first;               // > 0: keys j < keep_first are seen from any distance
};

#define AG_WARPS 4

__global__ void __launch_bounds__(AG_WARPS * 32) attention_generic_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * AG_WARPS + wib;
    if (w >= (long long)a.n_tokens * a.n_q) return;            // whole warps leave; no block barrier below
    const int t = (int)(w / a.n_q), head = (int)(w % a.n_q);
    const int g = head / (a.n_q / a.n_kv);
    float* qs = smem + wib * a.hd;
    const T* qrow = a.q + ((size_t)t * a.n_q + head) * a.hd;
    for (int d = lane; d < a.hd; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();
    const int pos = a.positions[t], s = a.token_seq[t], slot = a.slots[s];
    const int first_new = a.k_new ? a.q_start[s] : 0x7fffffff, tok0 = a.cu_q[s];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    // a sink is a key of score sink[head] (not scaled) whose value is zero: the sums start from it
    float m = a.sink ? a.sink[head] : -INFINITY, l = a.sink ? 1.f : 0.f;
    float acc[IDM_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
    const int keep = a.window > 0 ? min(a.keep_first, lo) : 0;     // kept keys below the window's first
    const int lo0 = (lo / 32) * 32, keep_end = min(((keep + 31) / 32) * 32, lo0);
    for (int j0 = keep > 0 ? 0 : lo0; j0 <= pos; j0 += 32) {
        if (j0 == keep_end && j0 < lo0) j0 = lo0;               // from the kept keys' last block on to the window's first
        const int j = j0 + lane;
        const bool valid = (j >= lo || j < keep) && j <= pos;
        float sc = -INFINITY;
        const T* vrow = nullptr;
        if (valid) {
            const T* krow;
            if (j >= first_new) {
                const size_t row = (size_t)(tok0 + j - first_new) * a.n_kv + g;
                krow = a.k_new + row * a.hd; vrow = a.v_new + row * a.dv;
            } else {
                const size_t row = kv_row(a.cache, slot, j, g);
                krow = a.cache.k + row * a.hd; vrow = a.cache.v + row * a.dv;
            }
            float dot = 0.f;
            if (a.hd % Vec16<T>::N == 0) {
                for (int d = 0; d < a.hd; d += Vec16<T>::N) {
                    Vec16<T> kv; kv.load(krow + d);
#pragma unroll
                    for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(qs[d + e], kv.get(e), dot);
                }
            } else {                                  // rows that do not start on 16-byte borders: the same sum, element by element
                for (int d = 0; d < a.hd; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
            }
            sc = dot * a.scale;
            if (a.softcap > 0.f) sc = a.softcap * tanhf(sc / a.softcap);
            if (a.slopes) sc -= a.slopes[head] * (float)(pos - j);
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float alpha = expf(m - m_new);
        const float p = valid ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] *= alpha;
        const unsigned live = __ballot_sync(0xffffffffu, valid);
        for (int jj = 0; jj < 32; ++jj) {
            if (!((live >> jj) & 1u)) continue;
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
#pragma unroll
            for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < a.dv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* orow = a.out + (size_t)t * a.out_stride + a.out_col + (size_t)head * a.dv;
    const float inv = 1.0f / l;
    const float* grow = a.gate && !a.gate_per_head ? a.gate + (size_t)t * a.gate_stride + (size_t)head * a.dv : nullptr;
    const float head_gate = a.gate && a.gate_per_head ? 1.0f / (1.0f + expf(-a.gate[(size_t)t * a.gate_stride + head])) : 1.f;
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.dv) {
            float o = acc[i] * inv * head_gate;
            if (grow) o = o / (1.0f + expf(-grow[d]));
            if (a.out_scale != 1.f) o *= a.out_scale;
            from_f32(orow[d], o);
        }
    }
}

static int attention_generic_launch(AttnArgs& a, cudaStream_t stream) {
    const long long warps = (long long)a.n_tokens * a.n_q;
    idm_launch(attention_generic_kernel, dim3((unsigned)((warps + AG_WARPS - 1) / AG_WARPS)), dim3(AG_WARPS * 32),
               AG_WARPS * a.hd * sizeof(float), stream, a);
    IDM_LAUNCH_CHECK("attention_generic");
    return 0;
}

extern "C" int idm_attention_generic(const void* q, void* out, void* k_pool, void* v_pool, const int* table,
                                     int table_stride, int ring, const void* k_new, const void* v_new,
                                     const int* token_seq, const int* positions, const int* slots,
                                     const int* q_start, const int* cu_q, int n_tokens, int n_q, int n_kv,
                                     int hd, float scale, int window, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd % Vec16<T>::N == 0 && hd <= IDM_MAX_HEAD_DIM,
                "attention: head_dim=%d must be a multiple of %d and at most %d", hd, Vec16<T>::N,
                IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d q-heads are no multiple of %d kv-heads", n_q, n_kv);
    IDM_REQUIRE((k_new == nullptr) == (v_new == nullptr), "attention: k_new and v_new come together");
    AttnArgs a;
    a.q = (const T*)q; a.out = (T*)out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.k_new = (const T*)k_new; a.v_new = (const T*)v_new;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.q_start = q_start; a.cu_q = cu_q;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd; a.scale = scale; a.window = window;
    a.dv = hd; a.sink = nullptr; a.gate = nullptr; a.gate_stride = 0; a.out_stride = n_q * hd; a.out_col = 0; a.out_scale = 1.f;
    a.slopes = nullptr; a.gate_per_head = 0; a.softcap = 0.f; a.keep_first = 0;
    return attention_generic_launch(a, stream);
}

// The same walk over the cache with what a gated attention with a sink adds: value rows of their own width
// `dv`, a learned score per head that joins the softmax's denominator without a key or a value, and the
// result times sigmoid(gate) times a constant, stored at a column offset of a wider buffer (gate: 32-bit
// [N, gate_stride], columns head * dv + d).  All keys come from the cache.
extern "C" int idm_attention_sink(const void* q, void* out, int out_stride, int out_col, float out_scale,
                                  void* k_pool, void* v_pool, const int* table, int table_stride,
                                  const float* sink, const float* gate, int gate_stride,
                                  const int* token_seq, const int* positions, const int* slots,
                                  const int* q_start, const int* cu_q, int n_tokens, int n_q, int n_kv,
                                  int hd, int dv, float scale, int window, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd <= IDM_MAX_HEAD_DIM && dv > 0 && dv <= IDM_MAX_HEAD_DIM,
                "attention: key and value sizes %d, %d must be at most %d", hd, dv, IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d q-heads are no multiple of %d kv-heads", n_q, n_kv);
    IDM_REQUIRE(out_col >= 0 && out_col + n_q * dv <= out_stride, "attention: columns %d..%d of rows of %d", out_col,
                out_col + n_q * dv, out_stride);
    AttnArgs a;
    a.q = (const T*)q; a.out = (T*)out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, 0, n_kv, hd};
    a.k_new = nullptr; a.v_new = nullptr;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.q_start = q_start; a.cu_q = cu_q;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd; a.scale = scale; a.window = window;
    a.dv = dv; a.sink = sink; a.gate = gate; a.gate_stride = gate_stride; a.out_stride = out_stride; a.out_col = out_col;
    a.out_scale = out_scale;
    a.slopes = nullptr; a.gate_per_head = 0; a.softcap = 0.f; a.keep_first = 0;
    return attention_generic_launch(a, stream);
}

// The same walk once more with every option this kernel has: a window over a cache that keeps all keys (ring 0) or
// a ring, a sink, a slope per head whose product with the distance p - j is taken off the score, a gate that is
// one number per head (gate_per_head) or one per channel, a cap on the scores and first keys that every query sees
// (keep_first; not with a ring, which does not keep them).
extern "C" int idm_attention_biased(const void* q, void* out, int out_stride, int out_col, float out_scale,
                                    void* k_pool, void* v_pool, const int* table, int table_stride, int ring,
                                    const float* sink, const float* slopes, const float* gate, int gate_stride,
                                    int gate_per_head, const int* token_seq, const int* positions, const int* slots,
                                    const int* q_start, const int* cu_q, int n_tokens, int n_q, int n_kv,
                                    int hd, int dv, float scale, int window, float softcap, int keep_first,
                                    cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd <= IDM_MAX_HEAD_DIM && dv > 0 && dv <= IDM_MAX_HEAD_DIM,
                "attention: key and value sizes %d, %d must be at most %d", hd, dv, IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d q-heads are no multiple of %d kv-heads", n_q, n_kv);
    IDM_REQUIRE(out_col >= 0 && out_col + n_q * dv <= out_stride, "attention: columns %d..%d of rows of %d", out_col,
                out_col + n_q * dv, out_stride);
    IDM_REQUIRE(keep_first >= 0 && softcap >= 0.f && (keep_first == 0 || ring == 0),
                "attention: keep_first=%d softcap=%g ring=%d (a ring does not keep a sequence's first keys)", keep_first, softcap, ring);
    AttnArgs a;
    a.q = (const T*)q; a.out = (T*)out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.k_new = nullptr; a.v_new = nullptr;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.q_start = q_start; a.cu_q = cu_q;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd; a.scale = scale; a.window = window;
    a.dv = dv; a.sink = sink; a.gate = gate; a.gate_stride = gate_stride; a.out_stride = out_stride; a.out_col = out_col;
    a.out_scale = out_scale; a.slopes = slopes; a.gate_per_head = gate_per_head;
    a.softcap = softcap; a.keep_first = keep_first;
    return attention_generic_launch(a, stream);
}
