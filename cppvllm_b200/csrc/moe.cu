// Routed feed-forward (mixture of experts): the router, the experts of a few tokens, and the experts of many.
//
//   route_topk     : z = x Wr^T + b in float (x may be bf16; Wr and b are float); the `top` largest logits are chosen
//                    (of equal logits the lower index first) and weighted by the softmax over the chosen logits only:
//                    ids[t, k], weights[t, k], k in order of falling logit.  One warp per token.
//   An expert is  Wd_e ( T(act(Wg_e x) * (Wu_e x)) ),  act(z) = z * sigmoid(z);  the layer's output is
//   y[t] = T( sum_k weights[t, k] * expert_{ids[t, k]}(x[t]) ).  Wgu is [E, 2 ff, D] (gate rows over up rows), Wd is
//   [E, D, ff].  Products and the weighted sum are float; the gated activation is rounded to T once, as the input of a
//   product.
//   A few tokens (decode; also the float path): two kernels that read only the chosen experts' weights, which is what
//   bounds such a step, with the work of a (token, expert) pair spread over many blocks so that every SM streams:
//     expert_hidden : block (pair, slice of ff): a warp owns inner elements, its lanes a row of the gate and of the up weight
//     expert_down   : block (token, slice of D): walks the token's experts, a warp owns output elements
//   Many tokens (prompt portions, bf16): the (token, expert) pairs are sorted by expert on the device (sort_pairs: counts,
//   offsets, a permutation; no trip to the host, so the step stays capturable), then two grouped products on the tensor
//   cores (grouped_gemm: tiles of 64 rows of ONE expert by 64 outputs, `mma.sync.m16n8k16` bf16 with float accumulation,
//   operands by cp.async into two stages; the rows of x are gathered through the permutation as they are loaded, so no
//   sorted copy of x exists; gate and up rows of the same inner elements share a tile, so the gated activation is the
//   epilogue), and a kernel that adds a token's expert outputs up with its weights.
#include "common.cuh"
#include "sm100.cuh"

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
constexpr int kExpertWarps = kExpertThreads / 32;

template <typename T> __device__ __forceinline__ float silu_exact(float g) { return g / (1.f + expf(-g)); }

// hid[pair, f] = T(silu(Wg_e[f] . x) * (Wu_e[f] . x)) for the block's slice of f; pair = t * top + k, e = ids[pair]
template <typename T>
__global__ void __launch_bounds__(kExpertThreads)
expert_hidden_kernel(T* __restrict__ hid, const T* __restrict__ x, const int* __restrict__ ids, const T* __restrict__ wgu,
                     int D, int F, int E, int top, int per_block, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* xs = smem;                                   // [D]
    const int64_t pair = blockIdx.x;
    const int64_t t = pair / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int e = ids[pair];
    if (e < 0 || e >= E) {
        if (threadIdx.x == 0) atomicExch(err, 7);
        e = 0;
    }
    for (int i = threadIdx.x; i < D; i += kExpertThreads) xs[i] = to_float(x[t * D + i]);
    __syncthreads();
    const T* g_rows = wgu + static_cast<int64_t>(e) * 2 * F * D;
    const T* u_rows = g_rows + static_cast<int64_t>(F) * D;
    const int f0 = blockIdx.y * per_block, f1 = min(F, f0 + per_block);
    for (int f = f0 + warp; f < f1; f += kExpertWarps) {
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
        if (lane == 0) hid[pair * F + f] = from_float<T>(silu_exact<T>(g) * u);
    }
}

// y[t, d] = T(sum_k weights[t, k] * (Wd_e[d] . hid[t * top + k])) for the block's slice of d
template <typename T>
__global__ void __launch_bounds__(kExpertThreads)
expert_down_kernel(T* __restrict__ y, const T* __restrict__ hid, const int* __restrict__ ids, const float* __restrict__ weights,
                   const T* __restrict__ wd, int D, int F, int E, int top, int per_block) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* hs = smem;                                   // [F]
    float* acc = hs + F;                                // [per_block]
    const int64_t t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d0 = blockIdx.y * per_block, d1 = min(D, d0 + per_block);
    for (int i = threadIdx.x; i < per_block; i += kExpertThreads) acc[i] = 0.f;
    for (int k = 0; k < top; ++k) {
        int e = ids[t * top + k];
        if (e < 0 || e >= E) e = 0;                      // reported by the kernel in front
        const float wk = weights[t * top + k];
        __syncthreads();
        for (int i = threadIdx.x; i < F; i += kExpertThreads) hs[i] = to_float(hid[(t * top + k) * F + i]);
        __syncthreads();
        const T* d_rows = wd + static_cast<int64_t>(e) * D * F;
        for (int d = d0 + warp; d < d1; d += kExpertWarps) {
            const T* dr = d_rows + static_cast<int64_t>(d) * F;
            float o = 0.f;
            for (int i = lane; i < F; i += 32) o = fmaf(hs[i], to_float(dr[i]), o);
            o = warp_sum(o);
            if (lane == 0) acc[d - d0] = fmaf(wk, o, acc[d - d0]);     // a warp owns its d: no other warp touches acc[d - d0]
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d1 - d0; i += kExpertThreads) y[t * D + d0 + i] = from_float<T>(acc[i]);
}

// ---- many tokens: pairs sorted by expert, grouped products on the tensor cores ------------------------------------------

constexpr int kSortThreads = 1024;

// counts per expert, offsets (exclusive prefix, [E + 1]), and the permutation: sorted[slot] = pair, slot_of[pair] = slot.
// One block.  The order of an expert's rows among themselves is not fixed; no result depends on it.
__global__ void __launch_bounds__(kSortThreads)
sort_pairs_kernel(int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ slot_of, const int* __restrict__ ids,
                  int n_pairs, int E, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int ismem[];
    int* count = ismem;                                 // [E]
    int* start = count + E;                             // [E + 1]
    for (int e = threadIdx.x; e < E; e += kSortThreads) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += kSortThreads) {
        int e = ids[i];
        if (e < 0 || e >= E) { atomicExch(err, 7); e = 0; }
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { start[e] = run; run += count[e]; }
        start[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += kSortThreads) offsets[e] = start[e];
    for (int e = threadIdx.x; e < E; e += kSortThreads) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_pairs; i += kSortThreads) {
        int e = ids[i];
        if (e < 0 || e >= E) e = 0;
        const int slot = start[e] + atomicAdd(&count[e], 1);
        sorted[slot] = i;
        slot_of[i] = slot;
    }
}

constexpr int kGemmThreads = 128;
constexpr int kGM = 64, kGN = 64, kGK = 32, kGLD = kGK + 8;

__device__ __forceinline__ void g_ldm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void g_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// out[r, n] for the sorted rows r of one expert e:  A row r is a[(gather ? gather[r] / top : r)] (K elements), B is expert
// e's matrix [N_rows, K] at b + e * b_stride.
//   GATED: the tile's 64 columns are 32 gate rows n0..n0+31 and the 32 up rows F + n0..; out[r, n0 + c] = silu(gate) * up
//   else : 64 rows n0..n0+63; out[r, n0 + c] = the product
// Block (tile of rows, slice of n).  Tiles are numbered expert by expert: ceil(count_e / 64) each; a block beyond the last
// tile returns.
template <bool GATED>
__global__ void __launch_bounds__(kGemmThreads)
grouped_gemm_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ a, const int* __restrict__ gather, int top,
                    const __nv_bfloat16* __restrict__ b, int64_t b_stride, const int* __restrict__ offsets, int E, int K, int N) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 sA[2][kGM * kGLD];
    __shared__ __align__(16) __nv_bfloat16 sB[2][kGN * kGLD];
    __shared__ int64_t a_row[kGM];
    int e = 0, tile = blockIdx.x, r0 = 0, r1 = 0;
    for (; e < E; ++e) {
        const int lo = offsets[e], n = offsets[e + 1] - lo;
        const int tiles = (n + kGM - 1) / kGM;
        if (tile < tiles) { r0 = lo + tile * kGM; r1 = min(lo + n, r0 + kGM); break; }
        tile -= tiles;
    }
    if (e >= E) return;
    const int n_out = GATED ? kGN / 2 : kGN;             // output columns of this block
    const int n0 = blockIdx.y * n_out;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int r = threadIdx.x; r < kGM; r += kGemmThreads) {
        const int row = r0 + r;
        a_row[r] = row < r1 ? static_cast<int64_t>(gather ? gather[row] / top : row) * K : -1;
    }
    __syncthreads();
    const __nv_bfloat16* be = b + static_cast<int64_t>(e) * b_stride;

    auto load = [&](int kt, int stage) {
        const int k0 = kt * kGK;
        for (int i = threadIdx.x; i < kGM * (kGK / 8); i += kGemmThreads) {
            const int r = i / (kGK / 8), c = i % (kGK / 8);
            const bool ok = a_row[r] >= 0 && k0 + c * 8 < K;
            cp_async16(&sA[stage][r * kGLD + c * 8], ok ? a + a_row[r] + k0 + c * 8 : a, ok);
        }
        for (int i = threadIdx.x; i < kGN * (kGK / 8); i += kGemmThreads) {
            const int r = i / (kGK / 8), c = i % (kGK / 8);
            int n;                                       // the weight row behind column r of the tile
            if (GATED) n = r < kGN / 2 ? n0 + r : N / 2 + n0 + (r - kGN / 2);
            else n = n0 + r;
            const bool in = GATED ? (n0 + (r % (kGN / 2)) < N / 2) : (n < N);
            const bool ok = in && k0 + c * 8 < K;
            cp_async16(&sB[stage][r * kGLD + c * 8], ok ? be + static_cast<int64_t>(n) * K + k0 + c * 8 : be, ok);
        }
    };

    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
    const int n_k = (K + kGK - 1) / kGK;
    load(0, 0);
    cp_async_commit();
    for (int kt = 0; kt < n_k; ++kt) {
        if (kt + 1 < n_k) load(kt + 1, (kt + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* tA = sA[kt & 1];
        const __nv_bfloat16* tB = sB[kt & 1];
#pragma unroll
        for (int ks = 0; ks < kGK / 16; ++ks) {
            uint32_t af[4];
            g_ldm_x4(af, tA + (warp * 16 + (lane & 15)) * kGLD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bf[4];
                g_ldm_x4(bf, tB + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * kGLD + ks * 16 + ((lane >> 3) & 1) * 8);
                g_mma(acc[np * 2], af, bf[0], bf[1]);
                g_mma(acc[np * 2 + 1], af, bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
    const int out_width = GATED ? N / 2 : N;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = r0 + warp * 16 + (lane >> 2) + half * 8;
        if (row >= r1) continue;
        __nv_bfloat16* dst = out + static_cast<int64_t>(row) * out_width;
#pragma unroll
        for (int nt = 0; nt < (GATED ? 4 : 8); ++nt) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int col = n0 + nt * 8 + ((lane & 3) << 1) + c;
                if (col >= out_width) continue;
                float v;
                if (GATED) {
                    const float g = acc[nt][half * 2 + c], u = acc[nt + 4][half * 2 + c];
                    v = g / (1.f + __expf(-g)) * u;
                } else {
                    v = acc[nt][half * 2 + c];
                }
                dst[col] = __float2bfloat16_rn(v);
            }
        }
    }
}

// y[t, :] = sum_k weights[t, k] * rows[slot_of[t * top + k], :]
__global__ void combine_pairs_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slot_of,
                                     const float* __restrict__ weights, int D, int top) {
    pdl_trigger();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k)
            s = fmaf(weights[t * top + k], __bfloat162float(rows[static_cast<int64_t>(slot_of[t * top + k]) * D + d]), s);
        y[t * D + d] = __float2bfloat16_rn(s);
    }
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

extern "C" int cvb_expert_rows(void* y, void* hid, const void* x, const int* ids, const float* weights, const void* wgu,
                               const void* wd, int T, int D, int F, int E, int top, int dtype, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || F <= 0 || E <= 0 || top <= 0) return CVB_E_SIZE;
    if (static_cast<size_t>(D) * sizeof(float) > 160 * 1024 || static_cast<size_t>(F) * sizeof(float) > 160 * 1024) return CVB_E_SIZE;
    // slices sized so that a step of one token still gives every SM a block or two
    const int64_t pairs = static_cast<int64_t>(T) * top;
    int f_per = kExpertWarps;
    while (pairs * ((F + f_per - 1) / f_per) > 1184 && f_per < F) f_per *= 2;
    int d_per = kExpertWarps;
    while (static_cast<int64_t>(T) * ((D + d_per - 1) / d_per) > 1184 && d_per < D) d_per *= 2;
    const size_t smem1 = static_cast<size_t>(D) * sizeof(float);
    const size_t smem2 = (static_cast<size_t>(F) + d_per) * sizeof(float);
    if (pairs > 2147483647LL / 2 || smem2 > 200 * 1024) return CVB_E_SIZE;
#define CALL(TY)                                                                                                         \
    do {                                                                                                                 \
        if (smem1 > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(expert_hidden_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);     \
        if (smem2 > 48 * 1024)                                                                                           \
            cudaFuncSetAttribute(expert_down_kernel<TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);       \
        launch_kernel(expert_hidden_kernel<TY>, dim3((unsigned)pairs, (F + f_per - 1) / f_per), dim3(kExpertThreads), smem1,  \
                      stream, (TY*)hid, (const TY*)x, ids, (const TY*)wgu, D, F, E, top, f_per, err_flag);                \
        launch_kernel(expert_down_kernel<TY>, dim3(T, (D + d_per - 1) / d_per), dim3(kExpertThreads), smem2, stream,      \
                      (TY*)y, (const TY*)hid, ids, weights, (const TY*)wd, D, F, E, top, d_per);                          \
    } while (0)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

// The grouped path (bf16): scratch `offsets` [E + 1], `sorted` and `slot_of` [T * top] ints, `hid` [T * top, F] and
// `rows` [T * top, D] bf16.
extern "C" int cvb_experts_grouped_bf16(void* y, const void* x, const int* ids, const float* weights, const void* wgu,
                                        const void* wd, int* offsets, int* sorted, int* slot_of, void* hid, void* rows, int T,
                                        int D, int F, int E, int top, int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || D <= 0 || F <= 0 || E <= 0 || top <= 0) return CVB_E_SIZE;
    if (D % 8 != 0 || F % 8 != 0) return CVB_E_ALIGN;
    const int64_t pairs64 = static_cast<int64_t>(T) * top;
    if (pairs64 > (1 << 30) || E > 4096) return CVB_E_SIZE;
    const int pairs = static_cast<int>(pairs64);
    launch_kernel(sort_pairs_kernel, dim3(1), dim3(kSortThreads), (2 * static_cast<size_t>(E) + 1) * sizeof(int), stream, offsets,
                  sorted, slot_of, ids, pairs, E, err_flag);
    const int max_tiles = (pairs + kGM - 1) / kGM + E;     // sum over experts of ceil(count / 64) never exceeds this
    launch_kernel(grouped_gemm_kernel<true>, dim3(max_tiles, (F + kGN / 2 - 1) / (kGN / 2)), dim3(kGemmThreads), 0, stream,
                  (__nv_bfloat16*)hid, (const __nv_bfloat16*)x, (const int*)sorted, top, (const __nv_bfloat16*)wgu,
                  static_cast<int64_t>(2) * F * D, (const int*)offsets, E, D, 2 * F);
    launch_kernel(grouped_gemm_kernel<false>, dim3(max_tiles, (D + kGN - 1) / kGN), dim3(kGemmThreads), 0, stream,
                  (__nv_bfloat16*)rows, (const __nv_bfloat16*)hid, (const int*)nullptr, 1, (const __nv_bfloat16*)wd,
                  static_cast<int64_t>(D) * F, (const int*)offsets, E, F, D);
    launch_kernel(combine_pairs_kernel, dim3(T), dim3(D >= 1024 ? 256 : 128), 0, stream, (__nv_bfloat16*)y,
                  (const __nv_bfloat16*)rows, (const int*)slot_of, weights, D, top);
    return launch_status();
}
