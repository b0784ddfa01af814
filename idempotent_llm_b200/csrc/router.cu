// A learned router over feed-forward experts: from a token's logits over all experts (identity experts included) to
// the experts it uses and their weights.
//
//   s      = softmax(z)                                   over all E experts, 32-bit
//   c_e    = s_e + correction_e                           the score an expert is CHOSEN by
//   groups : E / count neighbours each; a group's score is its largest c; only experts of the `keep` best groups
//            can be chosen (the others count as minus infinity)
//   chosen : the `top` largest c among those, in descending order (ties: the lower index)
//   weight : s_chosen / (sum of the chosen s + 1e-20) * scale
//
// One warp per token; s and c wait in shared memory.  Nothing here depends on the other tokens of the step.
#include "common.cuh"

#define RT_WARPS 4

// the lane holding the largest value (ties: the lowest index) tells everybody value and index
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

__global__ void __launch_bounds__(RT_WARPS * 32) route_kernel(const float* __restrict__ z, int z_stride,
                                                              const float* __restrict__ correction, int* __restrict__ chosen,
                                                              float* __restrict__ weight, int n_tokens, int E, int top,
                                                              int count, int keep, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RT_WARPS + wib;
    if (t >= n_tokens) return;                                   // whole warps leave; no block barrier below
    float* s = sm + (size_t)wib * (2 * E + count);               // [E] softmax
    float* c = s + E;                                            // [E] choice scores (minus infinity once taken or shut out)
    float* gs = c + E;                                           // [count] group scores
    const float* zr = z + (size_t)t * z_stride;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
    m = warp_max(m);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(zr[e] - m); s[e] = p; den += p; }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) { s[e] = s[e] / den; c[e] = s[e] + (correction ? correction[e] : 0.f); }
    __syncwarp();
    if (count > 1 && keep < count) {
        const int per = E / count;
        for (int g = lane; g < count; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
            gs[g] = best;
        }
        __syncwarp();
        // the `keep` best groups, one after another; gs of a kept group becomes +infinity as its mark
        for (int k = 0; k < keep; ++k) {
            float v = -INFINITY; int idx = 0x7fffffff;
            for (int g = lane; g < count; g += 32)
                if (gs[g] != INFINITY && (gs[g] > v || idx == 0x7fffffff)) { v = gs[g]; idx = g; }
            warp_argmax(v, idx);
            if (lane == 0 && idx != 0x7fffffff) gs[idx] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) c[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float v = -INFINITY; int idx = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (c[e] > v) { v = c[e]; idx = e; }                 // (ascending e: the lowest index of equal scores stays)
        warp_argmax(v, idx);
        if (idx == 0x7fffffff) idx = -1;                         // fewer experts open than `top`: the pair names no expert
        if (lane == 0) {
            chosen[(size_t)t * top + k] = idx;
            weight[(size_t)t * top + k] = idx >= 0 ? s[idx] : 0.f;
            if (idx >= 0) c[idx] = -INFINITY;
        }
        if (idx >= 0) total += s[idx];
        __syncwarp();
    }
    const float f = scale / (total + 1e-20f);
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= f;
}

extern "C" int idm_route(const float* z, int z_stride, const float* correction, int* chosen, float* weight, int n_tokens,
                         int n_experts, int top, int groups, int keep, float scale, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(n_experts > 0 && top > 0 && top <= n_experts && z_stride >= n_experts, "route: %d experts, %d per token, rows of %d",
                n_experts, top, z_stride);
    IDM_REQUIRE(groups >= 1 && n_experts % groups == 0 && keep >= 1 && keep <= groups, "route: %d experts in %d groups of which %d are kept",
                n_experts, groups, keep);
    const size_t smem = (size_t)RT_WARPS * (2 * n_experts + groups) * sizeof(float);
    IDM_REQUIRE(smem <= 160 * 1024, "route: %d experts do not fit shared memory", n_experts);
    if (smem > 48 * 1024) cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(route_kernel, dim3((n_tokens + RT_WARPS - 1) / RT_WARPS), dim3(RT_WARPS * 32), smem, stream, z, z_stride, correction,
               chosen, weight, n_tokens, n_experts, top, groups, keep, scale);
    IDM_LAUNCH_CHECK("route");
    return 0;
}

// h[t] += (sum of the weights of t's pairs that name an identity expert, chosen >= n_real) * x[t]
__global__ void __launch_bounds__(256) experts_identity_kernel(const T* __restrict__ x, const int* __restrict__ chosen,
                                                               const float* __restrict__ weight, float* __restrict__ h, int width,
                                                               int top, int n_real) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    float wsum = 0.f;
    for (int k = 0; k < top; ++k)
        if (chosen[t * top + k] >= n_real) wsum += weight[t * top + k];
    if (wsum == 0.f) return;
    for (int d = threadIdx.x; d < width; d += blockDim.x) h[t * width + d] = fmaf(wsum, to_f32(x[t * width + d]), h[t * width + d]);
}

extern "C" int idm_experts_identity(const void* x, const int* chosen, const float* weight, float* h, int n_tokens, int width,
                                    int top, int n_real, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    idm_launch(experts_identity_kernel, dim3(n_tokens), dim3(256), 0, stream, (const T*)x, chosen, weight, h, width, top, n_real);
    IDM_LAUNCH_CHECK("experts_identity");
    return 0;
}
