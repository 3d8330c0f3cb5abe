// Mixers that carry a state of fixed size per request instead of keys and values: the recurrence
//
//     S_t = a_t S_(t-1) + b_t k_t v_t^T        (S: dk x dv per head, 32-bit, in the request's state slot)
//     o_t = S_t^T q_t + D v_t
//
// with its two families of decay: a constant a per head and b = 1 (linear attention with decay), and
// a_t = exp(-exp(A_log) dt_t), b_t = dt_t with dt_t = softplus(raw_t + bias) per head and token (state-space
// duality). Around it: the short causal convolution over a request's tokens whose last inputs are state too,
// and the unit-RMS norm over groups of channels with a gate before (SiLU) or after (sigmoid) the norm.
//
// A step's rows are segments (one per request: seg_start, seg_len, state_slots as the step's descriptor holds
// them on the device). Tokens of a segment are taken in order, one after the other, by the same threads with the
// same arithmetic however the request was cut into steps and whatever else is in the batch; decays, step sizes,
// gates, norms and the state are 32-bit.
#include "common.cuh"

namespace gi {

__device__ __forceinline__ float silu_f(float z) { return z * (1.0f / (1.0f + expf(-z))); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------- causal convolution
// out[t, c] = silu(bias[c] + sum_j w[c, j] * u(t - (taps-1) + j, c)); u before the segment's first row is the
// request's conv state [taps-1, C] (oldest first; zeros for a new request), u before the sequence is zero.
__global__ void __launch_bounds__(256)
causal_conv_kernel(const float* __restrict__ in, int ld, int in_off, const float* __restrict__ weight,
                   const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                   const int* __restrict__ row_req, const int* __restrict__ seg_start,
                   const int* __restrict__ state_slots, float* __restrict__ out, int C, int taps, int T) {
    pdl_prologue();
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= C) return;
    const int r = row_req[t];
    const int rel = t - seg_start[r];
    const float* st = state + static_cast<long long>(state_slots[r]) * slot_stride;
    float acc = bias[c];
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                 // how many tokens before t
        float u;
        if (back <= rel) u = in[static_cast<size_t>(t - back) * ld + in_off + c];
        else u = st[static_cast<size_t>(taps - 1 + rel - back) * C + c];
        acc = fmaf(weight[static_cast<size_t>(c) * taps + j], u, acc);
    }
    out[static_cast<size_t>(t) * C + c] = silu_f(acc);
}

// The state after the step: the last taps-1 inputs of each segment (older ones from the old state).
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ in, int ld, int in_off, float* __restrict__ state, long long slot_stride,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                         const int* __restrict__ state_slots, int C, int taps) {
    pdl_prologue();
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= C) return;
    const int n = seg_len[r], s0 = seg_start[r];
    float* st = state + static_cast<long long>(state_slots[r]) * slot_stride;
    const int keep = taps - 1;
    float vals[16];
    for (int j = 0; j < keep; ++j) {
        const int rel = n - keep + j;                 // index among the segment's rows; negative: old state
        vals[j] = rel >= 0 ? in[static_cast<size_t>(s0 + rel) * ld + in_off + c] : st[static_cast<size_t>(keep + rel) * C + c];
    }
    for (int j = 0; j < keep; ++j) st[static_cast<size_t>(j) * C + c] = vals[j];
}

// ---------------------------------------------------------------------------------- the recurrence
// A block owns 32 columns of one head's state of one request; kSplit neighbouring lanes share a column, each with
// kRows of its rows in registers. Tokens are staged kChunk at a time in shared memory (activated, with their a and b).
constexpr int kScanCols = 32;
constexpr int kScanChunk = 16;

struct ScanArgs {
    const float* q; const float* k; const float* v;      // rows of ld_q / ld_k / ld_v floats, at these column offsets
    int ld_q, ld_k, ld_v, q_off, k_off, v_off;
    int H, group;                                         // head h reads q/k head h / group
    int dk, dv;
    int act;                                              // 1: SiLU on q, k and v when they are read
    const float* decay;                                   // [H] constant decays, or null for the dt form
    const float* dt_raw; int ld_dt, dt_off;               // [T, ld_dt] at dt_off + h
    const float* dt_bias; const float* a_log; const float* skip;      // [H] each; skip may be null
    float* state; long long slot_stride; long long state_off;          // per slot: [H, dk, dv] at state_off
    const int* seg_start; const int* seg_len; const int* state_slots;
    float* out;                                           // [T, H * dv]
};

template <int kRows, int kSplit>
__global__ void __launch_bounds__(kScanCols * kSplit)
linear_scan_kernel(const ScanArgs p) {
    pdl_prologue();
    constexpr int kDk = kRows * kSplit;                   // padded state rows
    __shared__ float s_q[kScanChunk][kDk];
    __shared__ float s_k[kScanChunk][kDk];
    __shared__ float s_v[kScanChunk][kScanCols];
    __shared__ float s_a[kScanChunk], s_b[kScanChunk];
    const int tile = blockIdx.x, h = blockIdx.y, r = blockIdx.z;
    const int g = h / p.group;
    const int col = threadIdx.x / kSplit, part = threadIdx.x % kSplit;
    const int j = tile * kScanCols + col;                 // column of the state
    const bool live = j < p.dv;
    const int n = p.seg_len[r], s0 = p.seg_start[r];
    float* S = p.state + static_cast<long long>(p.state_slots[r]) * p.slot_stride + p.state_off +
               static_cast<long long>(h) * p.dk * p.dv;
    float s[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const int row = part * kRows + i;
        s[i] = (live && row < p.dk) ? S[static_cast<size_t>(row) * p.dv + j] : 0.f;
    }
    const float skip = p.skip ? p.skip[h] : 0.f;
    const float a_const = p.decay ? p.decay[h] : 0.f;
    const float neg_rate = p.decay ? 0.f : -expf(p.a_log[h]);
    const float bias = p.decay ? 0.f : p.dt_bias[h];
    const int nthreads = kScanCols * kSplit;
    for (int c0 = 0; c0 < n; c0 += kScanChunk) {
        const int m = min(kScanChunk, n - c0);
        __syncthreads();
        for (int e = threadIdx.x; e < m * kDk; e += nthreads) {
            const int tt = e / kDk, i = e % kDk;
            const size_t t = static_cast<size_t>(s0 + c0 + tt);
            float qv = 0.f, kv = 0.f;
            if (i < p.dk) {
                qv = p.q[t * p.ld_q + p.q_off + g * p.dk + i];
                kv = p.k[t * p.ld_k + p.k_off + g * p.dk + i];
                if (p.act) { qv = silu_f(qv); kv = silu_f(kv); }
            }
            s_q[tt][i] = qv;
            s_k[tt][i] = kv;
        }
        for (int e = threadIdx.x; e < m * kScanCols; e += nthreads) {
            const int tt = e / kScanCols, cc = e % kScanCols;
            const int jj = tile * kScanCols + cc;
            float vv = 0.f;
            if (jj < p.dv) {
                vv = p.v[static_cast<size_t>(s0 + c0 + tt) * p.ld_v + p.v_off + h * p.dv + jj];
                if (p.act) vv = silu_f(vv);
            }
            s_v[tt][cc] = vv;
        }
        if (threadIdx.x < m) {
            if (p.decay) {
                s_a[threadIdx.x] = a_const;
                s_b[threadIdx.x] = 1.f;
            } else {
                const float dt = softplus_f(p.dt_raw[static_cast<size_t>(s0 + c0 + threadIdx.x) * p.ld_dt + p.dt_off + h] + bias);
                s_a[threadIdx.x] = expf(neg_rate * dt);
                s_b[threadIdx.x] = dt;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < m; ++tt) {
            const float a = s_a[tt], vj = s_v[tt][col];
            const float bv = s_b[tt] * vj;
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const int row = part * kRows + i;
                s[i] = fmaf(a, s[i], s_k[tt][row] * bv);
                o = fmaf(s[i], s_q[tt][row], o);
            }
#pragma unroll
            for (int w = kSplit / 2; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
            if (part == 0 && live)
                p.out[static_cast<size_t>(s0 + c0 + tt) * p.H * p.dv + h * p.dv + j] = fmaf(skip, vj, o);
        }
    }
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        const int row = part * kRows + i;
        if (live && row < p.dk) S[static_cast<size_t>(row) * p.dv + j] = s[i];
    }
}

// ---------------------------------------------------------------------------------- gated group norm
// One block per (token, group). mode 0: out = w * unit_rms(y) * sigmoid(gate); mode 1: out = w * unit_rms(y * silu(gate)).
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int ld_gate, int gate_off,
                        const float* __restrict__ weight, TOut* __restrict__ out, int W, int groups, float eps,
                        int mode, float out_scale) {
    pdl_prologue();
    __shared__ float warp_part[8];
    const int t = blockIdx.x, grp = blockIdx.y;
    const int n = W / groups;
    const float* yr = y + static_cast<size_t>(t) * W + grp * n;
    const float* gr = gate + static_cast<size_t>(t) * ld_gate + gate_off + grp * n;
    float ss = 0.f;
    for (int d = threadIdx.x; d < n; d += 256) {
        const float v = mode == 1 ? yr[d] * silu_f(gr[d]) : yr[d];
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += warp_part[w];
    const float scale = 1.0f / sqrtf(total / static_cast<float>(n) + eps);
    TOut* o = out + static_cast<size_t>(t) * W + grp * n;
    const float* w = weight + grp * n;
    for (int d = threadIdx.x; d < n; d += 256) {
        float v;
        if (mode == 1) v = w[d] * (scale * (yr[d] * silu_f(gr[d])));
        else v = w[d] * (scale * yr[d]) * (1.0f / (1.0f + expf(-gr[d])));
        o[d] = from_float<TOut>(v * out_scale);
    }
}

}  // namespace gi

using namespace gi;

static int gi_causal_conv_impl(const float* in, int ld, int in_off, const float* weight, const float* bias, float* state,
                               long long slot_stride, long long state_off, const int* row_req, const int* seg_start,
                               const int* seg_len, const int* state_slots, float* out, int C, int taps, int T, int R,
                               void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && R > 0 && C > 0, "causal_conv: sizes must be positive");
    GI_REQUIRE(taps >= 1 && taps <= 17, "causal_conv: %d taps are not supported (1 to 17)", taps);
    GI_REQUIRE(T <= 65535 && R <= 65535, "causal_conv: %d rows in one step exceed the grid limit 65535", T);
    GI_REQUIRE(in_off >= 0 && in_off + C <= ld, "causal_conv: the channels lie outside the input row of %d", ld);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned cb = (C + 255) / 256;
    launch_kernel((causal_conv_kernel), dim3(cb, T), dim3(256), 0, st, in, ld, in_off, weight, bias,
                  static_cast<const float*>(state + state_off), slot_stride, row_req, seg_start, state_slots, out, C, taps, T);
    if (taps > 1)
        launch_kernel((conv_state_update_kernel), dim3(cb, R), dim3(256), 0, st, in, ld, in_off, state + state_off, slot_stride,
                      seg_start, seg_len, state_slots, C, taps);
    return check_launch("causal_conv");
}

template <int kRows, int kSplit>
static void launch_scan(const ScanArgs& a, int R, cudaStream_t st) {
    dim3 grid((a.dv + kScanCols - 1) / kScanCols, a.H, R);
    launch_kernel((linear_scan_kernel<kRows, kSplit>), dim3(grid), dim3(kScanCols * kSplit), 0, st, a);
}

static int gi_linear_scan_impl(const float* q, int ld_q, int q_off, const float* k, int ld_k, int k_off, const float* v,
                               int ld_v, int v_off, int H, int group, int dk, int dv, int act, const float* decay,
                               const float* dt_raw, int ld_dt, int dt_off, const float* dt_bias, const float* a_log,
                               const float* skip, float* state, long long slot_stride, long long state_off,
                               const int* seg_start, const int* seg_len, const int* state_slots, float* out, int R,
                               void* stream) {
    if (R == 0) return 0;
    GI_REQUIRE(R > 0 && H > 0 && dk > 0 && dv > 0 && group > 0, "linear_scan: sizes must be positive");
    GI_REQUIRE(H % group == 0, "linear_scan: %d heads are not a multiple of the group size %d", H, group);
    GI_REQUIRE(dk <= 256, "linear_scan: %d state rows per head exceed 256", dk);
    GI_REQUIRE(R <= 65535 && H <= 65535, "linear_scan: the grid limit 65535 is exceeded");
    GI_REQUIRE(decay != nullptr || (dt_raw != nullptr && dt_bias != nullptr && a_log != nullptr),
               "linear_scan: neither constant decays nor step sizes are given");
    ScanArgs a{q, k, v, ld_q, ld_k, ld_v, q_off, k_off, v_off, H, group, dk, dv, act, decay, dt_raw, ld_dt, dt_off, dt_bias,
               a_log, skip, state, slot_stride, state_off, seg_start, seg_len, state_slots, out};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dk <= 16) launch_scan<4, 4>(a, R, st);
    else if (dk <= 32) launch_scan<8, 4>(a, R, st);
    else if (dk <= 64) launch_scan<16, 4>(a, R, st);
    else if (dk <= 128) launch_scan<32, 4>(a, R, st);
    else launch_scan<32, 8>(a, R, st);
    return check_launch("linear_scan");
}

static int gi_gated_group_norm_impl(const float* y, const float* gate, int ld_gate, int gate_off, const float* weight, void* out,
                                    int out_dtype, int T, int W, int groups, float eps, int mode, float out_scale, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && W > 0 && groups > 0 && W % groups == 0, "gated_group_norm: %d channels do not split into %d groups", W, groups);
    GI_REQUIRE(T <= 2147483647 && groups <= 65535, "gated_group_norm: the grid limit is exceeded");
    GI_REQUIRE(mode == 0 || mode == 1, "gated_group_norm: unknown mode %d", mode);
    GI_REQUIRE(gate_off >= 0 && gate_off + W <= ld_gate, "gated_group_norm: the gate lies outside its row of %d", ld_gate);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == kBF16)
        launch_kernel((gated_group_norm_kernel<__nv_bfloat16>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight,
                      static_cast<__nv_bfloat16*>(out), W, groups, eps, mode, out_scale);
    else if (out_dtype == kF32)
        launch_kernel((gated_group_norm_kernel<float>), dim3(T, groups), dim3(256), 0, st, y, gate, ld_gate, gate_off, weight,
                      static_cast<float*>(out), W, groups, eps, mode, out_scale);
    else
        GI_REQUIRE(false, "gated_group_norm: unsupported output dtype code %d", out_dtype);
    return check_launch("gated_group_norm");
}

extern "C" int gi_causal_conv(const float* in, int ld, int in_off, const float* weight, const float* bias, float* state, long long slot_stride, long long state_off, const int* row_req, const int* seg_start, const int* seg_len, const int* state_slots, float* out, int C, int taps, int T, int R, void* stream) {
    return gi::dispatch(gi_causal_conv_impl, in, ld, in_off, weight, bias, state, slot_stride, state_off, row_req, seg_start, seg_len, state_slots, out, C, taps, T, R, stream);
}

extern "C" int gi_linear_scan(const float* q, int ld_q, int q_off, const float* k, int ld_k, int k_off, const float* v, int ld_v, int v_off, int H, int group, int dk, int dv, int act, const float* decay, const float* dt_raw, int ld_dt, int dt_off, const float* dt_bias, const float* a_log, const float* skip, float* state, long long slot_stride, long long state_off, const int* seg_start, const int* seg_len, const int* state_slots, float* out, int R, void* stream) {
    return gi::dispatch(gi_linear_scan_impl, q, ld_q, q_off, k, ld_k, k_off, v, ld_v, v_off, H, group, dk, dv, act, decay, dt_raw, ld_dt, dt_off, dt_bias, a_log, skip, state, slot_stride, state_off, seg_start, seg_len, state_slots, out, R, stream);
}

extern "C" int gi_gated_group_norm(const float* y, const float* gate, int ld_gate, int gate_off, const float* weight, void* out, int out_dtype, int T, int W, int groups, float eps, int mode, float out_scale, void* stream) {
    return gi::dispatch(gi_gated_group_norm_impl, y, gate, ld_gate, gate_off, weight, out, out_dtype, T, W, groups, eps, mode, out_scale, stream);
}
