// Mixers that carry a matrix of fixed size per request and head from token to token instead of a cache that grows:
//
//   lightning_scan : q = silu(a_q), k = silu(a_k), v = silu(a_v) from a packed projection;  S <- d_h S + k v^T;  o = S^T q
//   delta_prep     : per token, everything the delta rule needs, in float: short causal convolutions over time (per channel,
//                    the last tap on the current token, history from the request's state where the portion begins) with
//                    silu behind them; q and k made unit vectors per head (x / sqrt(sum x^2 + 1e-6); q also times
//                    dk^-1/2); b = sigmoid(.); the decay g = exp(-exp(A_h) softplus(a + dt)) per head and key channel
//   conv_history   : the last taps - 1 raw inputs of every request's portion become the history of its next one
//   delta_scan     : S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q      (query/key head h / (H / G))
//
// S is [dk, dv] per (request, head), float, in the request's state slot; portions of any length continue where the
// state stands, one token after the other in the same order of operations, so cutting a sequence changes no bit.
// A block owns 32 columns of S of one (request, head); four lanes share a column (rows r * 4 + lane part) and add their
// parts up by shuffles.  The tokens of a portion are staged through shared memory a few at a time.
#include "common.cuh"

namespace cvb {

constexpr int kScanThreads = 128;
constexpr int kScanCols = 32;
constexpr int kLightChunk = 16;
constexpr int kDeltaChunk = 8;

__device__ __forceinline__ float silu_of(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_of(float z) { return 1.f / (1.f + expf(-z)); }

template <typename T, int KPT>
__global__ void __launch_bounds__(kScanThreads)
lightning_scan_kernel(float* __restrict__ out, const T* __restrict__ packed, int stride, int q_off, int k_off, int v_off,
                      float* __restrict__ state, int64_t state_floats, const float* __restrict__ decay,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int num_slots, int H, int dk, int dv,
                      int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    constexpr int dkp = KPT * 4;
    float* qs = sm;                               // [chunk][dkp]
    float* ks = qs + kLightChunk * dkp;           // [chunk][dkp]
    float* vs = ks + kLightChunk * dkp;           // [chunk][32]
    const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kScanCols;
    const int tid = threadIdx.x, col = tid >> 2, part = tid & 3, j = j0 + col;
    const int begin = cu_seqlens[s], end = cu_seqlens[s + 1];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) atomicExch(err, 2);
        return;
    }
    float* st = state + static_cast<int64_t>(slot) * state_floats + static_cast<int64_t>(h) * dk * dv;
    float S[KPT];
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * 4 + part;
        S[r] = (i < dk && j < dv) ? st[static_cast<int64_t>(i) * dv + j] : 0.f;
    }
    const float d = decay[h];
    for (int t0 = begin; t0 < end; t0 += kLightChunk) {
        const int n = min(kLightChunk, end - t0);
        __syncthreads();
        for (int idx = tid; idx < n * dkp; idx += kScanThreads) {
            const int tt = idx / dkp, i = idx - tt * dkp;
            float qv = 0.f, kv = 0.f;
            if (i < dk) {
                const T* row = packed + static_cast<int64_t>(t0 + tt) * stride;
                qv = silu_of(to_float(row[q_off + h * dk + i]));
                kv = silu_of(to_float(row[k_off + h * dk + i]));
            }
            qs[idx] = qv;
            ks[idx] = kv;
        }
        for (int idx = tid; idx < n * kScanCols; idx += kScanThreads) {
            const int tt = idx / kScanCols, c = idx - tt * kScanCols;
            vs[idx] = (j0 + c < dv) ? silu_of(to_float(packed[static_cast<int64_t>(t0 + tt) * stride + v_off + h * dv + j0 + c])) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float v = vs[tt * kScanCols + col];
            const float* kq = ks + tt * dkp + part;
            const float* qq = qs + tt * dkp + part;
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < KPT; ++r) {
                S[r] = fmaf(d, S[r], kq[r * 4] * v);
                o = fmaf(S[r], qq[r * 4], o);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (part == 0 && j < dv) out[(static_cast<int64_t>(t0 + tt) * H + h) * dv + j] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * 4 + part;
        if (i < dk && j < dv) st[static_cast<int64_t>(i) * dv + j] = S[r];
    }
}

// One block per token.  Channels: q [G * dk], k [G * dk], v [H * dv], in this order both in the packed row (from
// column qkv_off on) and in the convolution weights [C, taps] and the history [taps - 1, C] (oldest first).
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
delta_prep_kernel(float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ vv, float* __restrict__ gg, float* __restrict__ bb,
                  const T* __restrict__ packed, int stride, int qkv_off, const float* __restrict__ conv_w, int taps,
                  const float* __restrict__ a, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                  const float* __restrict__ b, const float* __restrict__ state, int64_t state_floats, int64_t conv_off,
                  const int* __restrict__ seq_of_token, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                  int num_slots, int H, int G, int dk, int dv, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];                 // conv outputs of q and k: [2 * G * dk]
    const int64_t t = blockIdx.x;
    const int tid = threadIdx.x;
    const int s = seq_of_token[t];
    const int local = static_cast<int>(t) - cu_seqlens[s];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) atomicExch(err, 2);
        return;
    }
    const int QK = G * dk, C = 2 * QK + H * dv;
    const float* hist = state + static_cast<int64_t>(slot) * state_floats + conv_off;
    for (int c = tid; c < C; c += kScanThreads) {
        float acc = 0.f;
        for (int jt = 0; jt < taps; ++jt) {
            const int o = local - (taps - 1) + jt;          // which token of the portion this tap reads; negative: before it
            const float x = o >= 0 ? to_float(packed[(t - (taps - 1) + jt) * stride + qkv_off + c])
                                   : hist[static_cast<int64_t>(local + jt) * C + c];
            acc = fmaf(conv_w[static_cast<int64_t>(c) * taps + jt], x, acc);
        }
        const float y = silu_of(acc);
        if (c < 2 * QK) sm[c] = y;
        else vv[t * H * dv + (c - 2 * QK)] = y;
    }
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31;
    for (int grp = warp; grp < 2 * G; grp += kScanThreads / 32) {
        const float* x = sm + grp * dk;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        float inv = 1.f / sqrtf(ss + 1e-6f);
        float* dst;
        if (grp < G) { inv *= 1.f / sqrtf(static_cast<float>(dk)); dst = qn + (t * G + grp) * dk; }
        else dst = kn + (t * G + (grp - G)) * dk;
        for (int i = lane; i < dk; i += 32) dst[i] = x[i] * inv;
    }
    for (int i = tid; i < H * dk; i += kScanThreads) {
        const float z = a[t * H * dk + i] + dt_bias[i];
        const float sp = z > 20.f ? z : log1pf(expf(z));
        gg[t * H * dk + i] = expf(-expf(a_log[i / dk]) * sp);
    }
    for (int i = tid; i < H; i += kScanThreads) bb[t * H + i] = sigmoid_of(b[t * H + i]);
}

// One block per request; a thread owns a channel and walks its history from the oldest entry on, so that an entry is read
// before it is overwritten.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
conv_history_kernel(float* __restrict__ state, int64_t state_floats, int64_t conv_off, const T* __restrict__ packed, int stride,
                    int qkv_off, int C, int taps, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                    int num_slots) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x;
    const int begin = cu_seqlens[s], n = cu_seqlens[s + 1] - begin;
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots || n <= 0) return;
    float* hist = state + static_cast<int64_t>(slot) * state_floats + conv_off;
    for (int c = blockIdx.y * kScanThreads + threadIdx.x; c < C; c += gridDim.y * kScanThreads) {
        for (int m = 0; m < taps - 1; ++m) {
            const int o = n - (taps - 1) + m;               // token of the portion that becomes entry m
            hist[static_cast<int64_t>(m) * C + c] = o >= 0 ? to_float(packed[static_cast<int64_t>(begin + o) * stride + qkv_off + c])
                                                           : hist[static_cast<int64_t>(n + m) * C + c];
        }
    }
}

template <int KPT>
__global__ void __launch_bounds__(kScanThreads)
delta_scan_kernel(float* __restrict__ out, const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vv,
                  const float* __restrict__ gg, const float* __restrict__ bb, float* __restrict__ state, int64_t state_floats,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, int num_slots, int H, int G, int dk, int dv,
                  int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    constexpr int dkp = KPT * 4;
    float* qs = sm;                               // [chunk][dkp]
    float* ks = qs + kDeltaChunk * dkp;
    float* gs = ks + kDeltaChunk * dkp;
    float* vs = gs + kDeltaChunk * dkp;           // [chunk][32]
    float* bs = vs + kDeltaChunk * kScanCols;     // [chunk]
    const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * kScanCols;
    const int kvh = h / (H / G);
    const int tid = threadIdx.x, col = tid >> 2, part = tid & 3, j = j0 + col;
    const int begin = cu_seqlens[s], end = cu_seqlens[s + 1];
    const int slot = state_slots[s];
    if (slot < 0 || slot >= num_slots) {
        if (tid == 0) atomicExch(err, 2);
        return;
    }
    float* st = state + static_cast<int64_t>(slot) * state_floats + static_cast<int64_t>(h) * dk * dv;
    float S[KPT];
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * 4 + part;
        S[r] = (i < dk && j < dv) ? st[static_cast<int64_t>(i) * dv + j] : 0.f;
    }
    for (int t0 = begin; t0 < end; t0 += kDeltaChunk) {
        const int n = min(kDeltaChunk, end - t0);
        __syncthreads();
        for (int idx = tid; idx < n * dkp; idx += kScanThreads) {
            const int tt = idx / dkp, i = idx - tt * dkp;
            const int64_t tok = t0 + tt;
            qs[idx] = i < dk ? qn[(tok * G + kvh) * dk + i] : 0.f;
            ks[idx] = i < dk ? kn[(tok * G + kvh) * dk + i] : 0.f;
            gs[idx] = i < dk ? gg[(tok * H + h) * dk + i] : 0.f;
        }
        for (int idx = tid; idx < n * kScanCols; idx += kScanThreads) {
            const int tt = idx / kScanCols, c = idx - tt * kScanCols;
            vs[idx] = (j0 + c < dv) ? vv[(static_cast<int64_t>(t0 + tt) * H + h) * dv + j0 + c] : 0.f;
        }
        if (tid < n) bs[tid] = bb[static_cast<int64_t>(t0 + tid) * H + h];
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float* kq = ks + tt * dkp + part;
            const float* qq = qs + tt * dkp + part;
            const float* gq = gs + tt * dkp + part;
            float dot = 0.f;
#pragma unroll
            for (int r = 0; r < KPT; ++r) {
                S[r] *= gq[r * 4];
                dot = fmaf(S[r], kq[r * 4], dot);
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            const float u = bs[tt] * (vs[tt * kScanCols + col] - dot);
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < KPT; ++r) {
                S[r] = fmaf(kq[r * 4], u, S[r]);
                o = fmaf(S[r], qq[r * 4], o);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (part == 0 && j < dv) out[(static_cast<int64_t>(t0 + tt) * H + h) * dv + j] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
        const int i = r * 4 + part;
        if (i < dk && j < dv) st[static_cast<int64_t>(i) * dv + j] = S[r];
    }
}

}  // namespace cvb

using namespace cvb;

#define CVB_DISPATCH_KPT(dk, CALL)                  \
    do {                                            \
        if ((dk) <= 32) { CALL(8); }                \
        else if ((dk) <= 64) { CALL(16); }          \
        else if ((dk) <= 128) { CALL(32); }         \
        else { CALL(64); }                          \
    } while (0)

extern "C" int cvb_lightning_scan(float* out, const void* packed, int stride, int q_off, int k_off, int v_off, float* state,
                                  int64_t state_floats, const float* decay, const int* cu_seqlens, const int* state_slots,
                                  int num_slots, int S, int H, int dk, int dv, int dtype, int* err_flag, cudaStream_t stream) {
    if (S == 0) return CVB_OK;
    if (S < 0 || H <= 0 || H > 65535 || dk <= 0 || dk > 256 || dv <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (q_off < 0 || k_off < 0 || v_off < 0 || stride < H * dk || state_floats < static_cast<int64_t>(H) * dk * dv) return CVB_E_SHAPE;
    const dim3 grid(S, H, (dv + kScanCols - 1) / kScanCols);
#define CALL_K(KPT)                                                                                                        \
    do {                                                                                                                   \
        const size_t smem = (2 * kLightChunk * KPT * 4 + kLightChunk * kScanCols) * sizeof(float);                          \
        if (dtype == CVB_DTYPE_F32)                                                                                        \
            launch_kernel(lightning_scan_kernel<float, KPT>, grid, dim3(kScanThreads), smem, stream, out, (const float*)packed, \
                          stride, q_off, k_off, v_off, state, state_floats, decay, cu_seqlens, state_slots, num_slots, H, dk, dv, err_flag); \
        else if (dtype == CVB_DTYPE_BF16)                                                                                  \
            launch_kernel(lightning_scan_kernel<__nv_bfloat16, KPT>, grid, dim3(kScanThreads), smem, stream, out,          \
                          (const __nv_bfloat16*)packed, stride, q_off, k_off, v_off, state, state_floats, decay, cu_seqlens, \
                          state_slots, num_slots, H, dk, dv, err_flag);                                                    \
        else return CVB_E_DTYPE;                                                                                           \
    } while (0)
    CVB_DISPATCH_KPT(dk, CALL_K);
#undef CALL_K
    return launch_status();
}

extern "C" int cvb_delta_prep(float* qn, float* kn, float* vv, float* gg, float* bb, const void* packed, int T, int stride, int qkv_off,
                              const float* conv_w, int taps, const float* a, const float* dt_bias, const float* a_log, const float* b,
                              const float* state, int64_t state_floats, int64_t conv_off, const int* seq_of_token,
                              const int* cu_seqlens, const int* state_slots, int num_slots, int H, int G, int dk, int dv, int dtype,
                              int* err_flag, cudaStream_t stream) {
    if (T == 0) return CVB_OK;
    if (T < 0 || H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || taps <= 0 || num_slots <= 0) return CVB_E_SIZE;
    const int64_t C = 2LL * G * dk + static_cast<int64_t>(H) * dv;
    if (H % G || qkv_off < 0 || stride < qkv_off + C || state_floats < conv_off + (taps - 1) * C) return CVB_E_SHAPE;
    const size_t smem = static_cast<size_t>(2) * G * dk * sizeof(float);
    if (smem > 48 * 1024) return CVB_E_SIZE;
#define CALL(TY) launch_kernel(delta_prep_kernel<TY>, dim3(T), dim3(kScanThreads), smem, stream, qn, kn, vv, gg, bb, (const TY*)packed, \
                               stride, qkv_off, conv_w, taps, a, dt_bias, a_log, b, state, state_floats, conv_off, seq_of_token,       \
                               cu_seqlens, state_slots, num_slots, H, G, dk, dv, err_flag)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_conv_history(float* state, int64_t state_floats, int64_t conv_off, const void* packed, int stride, int qkv_off, int C,
                                int taps, const int* cu_seqlens, const int* state_slots, int num_slots, int S, int dtype,
                                cudaStream_t stream) {
    if (S == 0 || taps <= 1) return CVB_OK;
    if (S < 0 || C <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (qkv_off < 0 || stride < qkv_off + C || state_floats < conv_off + static_cast<int64_t>(taps - 1) * C) return CVB_E_SHAPE;
    const dim3 grid(S, (C + kScanThreads - 1) / kScanThreads);
#define CALL(TY) launch_kernel(conv_history_kernel<TY>, grid, dim3(kScanThreads), 0, stream, state, state_floats, conv_off, \
                               (const TY*)packed, stride, qkv_off, C, taps, cu_seqlens, state_slots, num_slots)
    CVB_DISPATCH_DTYPE(dtype, CALL);
#undef CALL
    return launch_status();
}

extern "C" int cvb_delta_scan(float* out, const float* qn, const float* kn, const float* vv, const float* gg, const float* bb,
                              float* state, int64_t state_floats, const int* cu_seqlens, const int* state_slots, int num_slots, int S,
                              int H, int G, int dk, int dv, int* err_flag, cudaStream_t stream) {
    if (S == 0) return CVB_OK;
    if (S < 0 || H <= 0 || H > 65535 || G <= 0 || dk <= 0 || dk > 256 || dv <= 0 || num_slots <= 0) return CVB_E_SIZE;
    if (H % G || state_floats < static_cast<int64_t>(H) * dk * dv) return CVB_E_SHAPE;
    const dim3 grid(S, H, (dv + kScanCols - 1) / kScanCols);
#define CALL_K(KPT)                                                                                                     \
    do {                                                                                                                \
        const size_t smem = (3 * kDeltaChunk * KPT * 4 + kDeltaChunk * kScanCols + kDeltaChunk) * sizeof(float);          \
        launch_kernel(delta_scan_kernel<KPT>, grid, dim3(kScanThreads), smem, stream, out, qn, kn, vv, gg, bb, state,   \
                      state_floats, cu_seqlens, state_slots, num_slots, H, G, dk, dv, err_flag);                        \
    } while (0)
    CVB_DISPATCH_KPT(dk, CALL_K);
#undef CALL_K
    return launch_status();
}
