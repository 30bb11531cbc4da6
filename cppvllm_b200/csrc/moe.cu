// Routed feed-forward (mixture of experts): the router, and the experts of a few tokens.
//
//   route_topk   : z = x Wr^T + b in float (x may be bf16; Wr and b are float); the `top` largest logits are chosen
//                  (of equal logits the lower index first) and weighted by the softmax over the chosen logits only:
//                  ids[t, k], weights[t, k], k in order of falling logit.  One warp per token.
//   expert_rows  : y[t] = T( sum_k weights[t, k] * ( Wd_e (T(act(Wg_e x) * (Wu_e x))) ) ),  e = ids[t, k],
//                  act(z) = z * sigmoid(z).  One block per token walks the token's experts; a warp owns an output element
//                  and its lanes a row of the weight (one coalesced read per row).  Only the chosen experts' weights are
//                  read, which is what bounds a step of a few tokens.  Wgu is [E, 2 ff, D] (gate rows over up rows),
//                  Wd is [E, D, ff].  Products and the weighted sum are float; the gated activation is rounded to T once,
//                  as the input of a product.
#include "common.cuh"

namespace cvb {

constexpr int kRouteWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
route_topk_kernel(int* __restrict__ ids, float* __restrict__ weights, const T* __restrict__ x, const float* __restrict__ wr,
                  const float* __restrict__ bias, int n_tokens, int D, int E, int top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];                     // [kRouteWarps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRouteWarps + warp;
    if (t >= n_tokens) return;
    float* z = smem + warp * E;
    const T* xr = x + t * D;
    for (int e = 0; e < E; ++e) {
        const float* w = wr + static_cast<int64_t>(e) * D;
        float d = 0.f;
        for (int i = lane; i < D; i += 32) d = fmaf(to_float(xr[i]), w[i], d);
        d = warp_sum(d);
        if (lane == 0) z[e] = d + (bias ? bias[e] : 0.f);
    }
    __syncwarp();
    float z_first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; at = e; }          // the lower index wins among a lane's equals
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) z_first = best;
        const float p = expf(best - z_first);
        sum += p;
        if (lane == 0) {
            ids[t * top + k] = at;
            weights[t * top + k] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.f / sum;
    for (int k = lane; k < top; k += 32) weights[t * top + k] *= inv;     // lane 0's writes are visible after the syncwarp
}

constexpr int kExpertThreads = 256;

template <typename T> __device__ __forceinline__ float silu_exact(float g) { return g / (1.f + expf(-g)); }

template <typename T>
__global__ void __launch_bounds__(kExpertThreads)
expert_rows_kernel(T* __restrict__ y, const T* __restrict__ x, const int* __restrict__ ids, const float* __restrict__ weights,
                   const T* __restrict__ wgu, const T* __restrict__ wd, int D, int F, int E, int top, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* xs = smem;                                   // [D]
    float* hid = xs + D;                                // [F]
    float* acc = hid + F;                               // [D]
    const int64_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = kExpertThreads / 32;
    for (int i = threadIdx.x; i < D; i += kExpertThreads) { xs[i] = to_float(x[t * D + i]); acc[i] = 0.f; }
    __syncthreads();
    for (int k = 0; k < top; ++k) {
        int e = ids[t * top + k];
        if (e < 0 || e >= E) {
            if (threadIdx.x == 0) atomicExch(err, 7);
            e = 0;
        }
        const float wk = weights[t * top + k];
        const T* g_rows = wgu + static_cast<int64_t>(e) * 2 * F * D;
        const T* u_rows = g_rows + static_cast<int64_t>(F) * D;
        for (int f = warp; f < F; f += n_warps) {
            const T* gr = g_rows + static_cast<int64_t>(f) * D;
            const T* ur = u_rows + static_cast<int64_t>(f) * D;
            float g = 0.f, u = 0.f;
            for (int i = lane; i < D; i += 32) {
                const float xv = xs[i];
                g = fmaf(xv, to_float(gr[i]), g);
                u = fmaf(xv, to_float(ur[i]), u);
            }
            g = warp_sum(g);
            u = warp_sum(u);
            if (lane == 0) hid[f] = rnd<T>(silu_exact<T>(g) * u);
        }
        __syncthreads();
        const T* d_rows = wd + static_cast<int64_t>(e) * D * F;
        for (int d = warp; d < D; d += n_warps) {
            const T* dr = d_rows + static_cast<int64_t>(d) * F;
            float o = 0.f;
            for (int i = lane; i < F; i += 32) o = fmaf(hid[i], to_float(dr[i]), o);
            o = warp_sum(o);
            if (lane == 0) acc[d] = fmaf(wk, o, acc[d]);
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < D; i += kExpertThreads) y[t * D + i] = from_float<T>(acc[i]);
}

}  // namespace cvb

using namespace cvb;

extern "C" int cvb_route_topk(int* ids, float* weights, const void* x, const float* wr, const float* bias, int T, int D, int E,
                              int top, int dtype, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || E <= 0 || top <= 0) return CVB_E_SIZE;
    if (top > E || E > 2048) return CVB_E_SHAPE;
    const size_t smem = static_cast<size_t>(kRouteWarps) * E * sizeof(float);
#define CALL(TY) launch_kernel(route_topk_kernel<TY>, dim3((T + kRouteWarps - 1) / kRouteWarps), dim3(kRouteWarps * 32), smem, \
                               stream, ids, weights, (const TY*)x, wr, bias, T, D, E, top)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_expert_rows(void* y, const void* x, const int* ids, const float* weights, const void* wgu, const void* wd,
                               int T, int D, int F, int E, int top, int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || F <= 0 || E <= 0 || top <= 0) return CVB_E_SIZE;
    const size_t smem = (2 * static_cast<size_t>(D) + F) * sizeof(float);
    if (smem > 200 * 1024) return CVB_E_SIZE;
#define CALL(TY)                                                                                                        \
    do {                                                                                                                \
        if (smem > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(expert_rows_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        launch_kernel(expert_rows_kernel<TY>, dim3(T), dim3(kExpertThreads), smem, stream, (TY*)y, (const TY*)x, ids,   \
                      weights, (const TY*)wgu, (const TY*)wd, D, F, E, top, err_flag);                                  \
    } while (0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}
