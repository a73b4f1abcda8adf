// A gated recurrence whose gates read only the current token (minGRU), element by element, and the blend of a token's
// input with the input of the token before it that RWKV-style mixers feed their projections with.
//
// gated_recurrence: rows [ ... z (W) ... u (W) ... g (W) ... ] of 32-bit pre-activations (biases included), per
// request r and channel c, over the request's tokens t in order:
//   s <- (1 - sigmoid(z_t)) s + sigmoid(z_t) cand(u_t),   cand(u) = u + 1/2 for u >= 0, sigmoid(u) below,
//   out_t = s * silu(g_t)
// s lives in the request's state slot in 32-bit and starts at zero when the request has nothing in the cache.  One
// thread owns a channel; a token is one multiply-add on the chain, everything else (the loads of eight tokens at a
// time, the logistic functions) does not wait for the state.  The order of the sums is the tokens' order whatever
// the cut into steps.
//
// gated_recurrence_ranges (long portions where the cut may move the last bits: bfloat16 steps): a CTA owns 8
// channels of one request (a quarter of a warp reads 32 bytes of a row: whole sectors) and its 128 quarter-warps
// share the request's tokens in equal ranges, so that width / 8 CTAs fill the GPU at widths of a thousand and more.
// The recurrence is affine in s, so a range is the pair (keep, add) with s_out = keep * s_in + add: every
// quarter-warp scans its range once from s = 0 with keep = prod (1 - z), the pairs meet in shared memory, it folds
// the pairs of the ranges before its own into its incoming state, and scans its range again from there, writing the
// outputs.  The chain is two passes over a range instead of one over the portion; state, gates and sums stay 32-bit.
//
// token_shift_mix: with h_t a token's input and h_(t-1) the input of the token before it in its sequence (zeros for a
// sequence's first token; for a step's first token of a request it is read from the request's state slot),
//   out[s][t] = h_t + (h_(t-1) - h_t) * mu[s]        for s = 0 .. n_mixes - 1
// conv_state_update of short_conv.cu with two taps leaves a step's last input in the slot afterwards.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(recurrent_gate)

namespace {

constexpr int THREADS = 128;
constexpr int AHEAD = 8;          // tokens whose rows are loaded before the chain runs over them

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(THREADS)
gated_recurrence_kernel(const float* __restrict__ pre, int ld, int z_off, int u_off, int g_off,
                        const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                        const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                        float* __restrict__ state, long long state_stride, T* __restrict__ out, int width, int n_slots,
                        int n_tokens) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, c = blockIdx.x * THREADS + threadIdx.x;
    const int q_len = req_q_len[r];
    if (q_len <= 0 || c >= width) return;                      // a padding row of a fixed-size batch
    const int start = req_q_start[r];
    int slot = req_state_slot[r];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_ROW, slot, n_slots) ||
        !MG_GUARDED(recurrent_gate, MG_GUARD_ROW, start + q_len - 1, n_tokens))
        return;
    float* s_ptr = state + (size_t)slot * state_stride + c;
    float s = req_ctx_before[r] == 0 ? 0.f : *s_ptr;
    for (int t0 = 0; t0 < q_len; t0 += AHEAD) {
        float zv[AHEAD], uv[AHEAD], gv[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const bool live = t0 + i < q_len;
            const float* row = pre + (size_t)(start + t0 + (live ? i : 0)) * ld + c;
            zv[i] = row[z_off];
            uv[i] = row[u_off];
            gv[i] = row[g_off];
        }
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            if (t0 + i >= q_len) break;
            const float z = sigmoidf(zv[i]);
            const float cand = uv[i] >= 0.f ? uv[i] + 0.5f : sigmoidf(uv[i]);
            s = fmaf(z, cand - s, s);                          // (1 - z) s + z cand
            out[(size_t)(start + t0 + i) * width + c] = from_float<T>(s * gv[i] * sigmoidf(gv[i]));
        }
    }
    *s_ptr = s;
}

constexpr int RANGE_WARPS = 32;   // warps of a CTA of the range form
constexpr int RANGE_CH = 8;       // channels a CTA owns: a quarter of a warp
constexpr int RANGES = RANGE_WARPS * (32 / RANGE_CH);   // token ranges a request is cut into

template <typename T>
__global__ void __launch_bounds__(32 * RANGE_WARPS)
gated_recurrence_ranges_kernel(const float* __restrict__ pre, int ld, int z_off, int u_off, int g_off,
                               const int* __restrict__ req_q_start, const int* __restrict__ req_q_len,
                               const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                               float* __restrict__ state, long long state_stride, T* __restrict__ out, int width,
                               int n_slots, int n_tokens) {
    __shared__ float keep_s[RANGES][RANGE_CH], add_s[RANGES][RANGE_CH];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, range = threadIdx.x / RANGE_CH, lane = threadIdx.x % RANGE_CH;
    const int c = blockIdx.x * RANGE_CH + lane;
    const int q_len = req_q_len[r];
    if (q_len <= 0) return;                                    // a padding row of a fixed-size batch
    const int start = req_q_start[r];
    int slot = req_state_slot[r];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_ROW, slot, n_slots) ||
        !MG_GUARDED(recurrent_gate, MG_GUARD_ROW, start + q_len - 1, n_tokens))
        return;
    const bool live = c < width;
    const int per = (q_len + RANGES - 1) / RANGES;
    const int t_begin = min(range * per, q_len), t_end = min(t_begin + per, q_len);
    const float* base = pre + (size_t)start * ld + (live ? c : 0);
    float keep = 1.f, add = 0.f;
    for (int t0 = t_begin; t0 < t_end; t0 += AHEAD) {
        float zv[AHEAD], uv[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const float* row = base + (size_t)min(t0 + i, t_end - 1) * ld;
            zv[i] = row[z_off];
            uv[i] = row[u_off];
        }
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            if (t0 + i >= t_end) break;
            const float z = sigmoidf(zv[i]);
            const float cand = uv[i] >= 0.f ? uv[i] + 0.5f : sigmoidf(uv[i]);
            add = fmaf(z, cand - add, add);
            keep *= 1.f - z;
        }
    }
    keep_s[range][lane] = keep;
    add_s[range][lane] = add;
    __syncthreads();
    float* s_ptr = state + (size_t)slot * state_stride + (live ? c : 0);
    float s = (req_ctx_before[r] == 0 || !live) ? 0.f : *s_ptr;
    for (int w = 0; w < range; ++w) s = fmaf(keep_s[w][lane], s, add_s[w][lane]);
    for (int t0 = t_begin; t0 < t_end; t0 += AHEAD) {
        float zv[AHEAD], uv[AHEAD], gv[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const float* row = base + (size_t)min(t0 + i, t_end - 1) * ld;
            zv[i] = row[z_off];
            uv[i] = row[u_off];
            gv[i] = row[g_off];
        }
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            if (t0 + i >= t_end) break;
            const float z = sigmoidf(zv[i]);
            const float cand = uv[i] >= 0.f ? uv[i] + 0.5f : sigmoidf(uv[i]);
            s = fmaf(z, cand - s, s);
            if (live) out[(size_t)(start + t0 + i) * width + c] = from_float<T>(s * gv[i] * sigmoidf(gv[i]));
        }
    }
    // the last range that holds tokens leaves the state
    if (live && t_end == q_len && t_begin < t_end) *s_ptr = s;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
token_shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, const int* __restrict__ token_request,
                       const int* __restrict__ positions, const int* __restrict__ req_q_start,
                       const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                       const float* __restrict__ state, long long state_stride, T* __restrict__ out, int width,
                       int n_mixes, int n_tokens, int n_requests, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, c = blockIdx.y * THREADS + threadIdx.x;
    if (c >= width) return;
    const size_t plane = (size_t)n_tokens * width, at = (size_t)token * width + c;
    if (positions[token] < 0) {                                // padding: nothing is read for it
        for (int s = 0; s < n_mixes; ++s) out[s * plane + at] = from_float<T>(0.f);
        return;
    }
    int r = token_request[token];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_REQUEST, r, n_requests)) return;
    int slot = req_state_slot[r];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_ROW, slot, n_slots)) return;
    const float cur = to_float(x[at]);
    float before;
    if (token > req_q_start[r]) before = to_float(x[at - width]);
    else before = req_ctx_before[r] == 0 ? 0.f : state[(size_t)slot * state_stride + c];
    const float diff = before - cur;
    for (int s = 0; s < n_mixes; ++s) out[s * plane + at] = from_float<T>(fmaf(diff, mu[(size_t)s * width + c], cur));
}

// The same with 16 bytes a load: a thread takes VEC neighbouring channels of a token (8 bfloat16 or 4 32-bit numbers).
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) { const float4 r = *reinterpret_cast<const float4*>(p); v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Pack<bf16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void load(const bf16* p) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int u = 0; u < 4; ++u) { v[2 * u] = __bfloat162float(h[u].x); v[2 * u + 1] = __bfloat162float(h[u].y); }
    }
    __device__ __forceinline__ void store(bf16* p) const {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int u = 0; u < 4; ++u) h[u] = __floats2bfloat162_rn(v[2 * u], v[2 * u + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

template <typename T>
__global__ void __launch_bounds__(THREADS)
token_shift_mix_vec_kernel(const T* __restrict__ x, const float* __restrict__ mu, const int* __restrict__ token_request,
                           const int* __restrict__ positions, const int* __restrict__ req_q_start,
                           const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                           const float* __restrict__ state, long long state_stride, T* __restrict__ out, int width,
                           int n_mixes, int n_tokens, int n_requests, int n_slots) {
    constexpr int N = Pack<T>::N;
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, c = (blockIdx.y * THREADS + threadIdx.x) * N;
    if (c >= width) return;
    const size_t plane = (size_t)n_tokens * width, at = (size_t)token * width + c;
    Pack<T> cur, before, res;
    if (positions[token] < 0) {                                // padding: nothing is read for it
#pragma unroll
        for (int u = 0; u < N; ++u) res.v[u] = 0.f;
        for (int s = 0; s < n_mixes; ++s) res.store(out + s * plane + at);
        return;
    }
    int r = token_request[token];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_REQUEST, r, n_requests)) return;
    int slot = req_state_slot[r];
    if (!MG_GUARDED(recurrent_gate, MG_GUARD_ROW, slot, n_slots)) return;
    cur.load(x + at);
    if (token > req_q_start[r]) {
        before.load(x + at - width);
    } else {
        const bool fresh = req_ctx_before[r] == 0;
        const float* old = state + (size_t)slot * state_stride + c;
#pragma unroll
        for (int u = 0; u < N; ++u) before.v[u] = fresh ? 0.f : old[u];
    }
    for (int s = 0; s < n_mixes; ++s) {
        const float* m = mu + (size_t)s * width + c;
#pragma unroll
        for (int u = 0; u < N; ++u) res.v[u] = fmaf(before.v[u] - cur.v[u], m[u], cur.v[u]);
        res.store(out + s * plane + at);
    }
}

}  // namespace

// pre: [n_tokens, ld] 32-bit rows holding z, u and g (width numbers each) at the three column offsets; req_*:
// [n_requests] first row, tokens, tokens already in the cache, state slot; state: 32-bit, `state_stride` numbers
// a slot, of which the first `width` (from `state`) are this recurrence's; out: [n_tokens, width].  ranges: 1 for
// the form whose warps share a request's tokens (sums in another order than token by token), 0 token by token.
MG_API int mg_gated_recurrence(const float* pre, int ld, int z_off, int u_off, int g_off, const int* req_q_start,
                               const int* req_q_len, const int* req_ctx_before, const int* req_state_slot, float* state,
                               long long state_stride, void* out, int n_requests, int n_tokens, int width, int n_slots,
                               int out_bf16, int ranges, void* stream) {
    if (n_requests == 0 || n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_requests > 0 && n_requests <= 65535 && n_tokens > 0 && width > 0 && n_slots > 0 && state_stride >= width,
               "gated recurrence: bad sizes");
    MG_REQUIRE(z_off >= 0 && u_off >= 0 && g_off >= 0 && z_off + width <= ld && u_off + width <= ld && g_off + width <= ld,
               "gated recurrence: columns outside the rows");
    cudaStream_t s = (cudaStream_t)stream;
    if (ranges) {                                              // long portions: the warps of a CTA share the tokens
        const dim3 rgrid(ceil_div(width, RANGE_CH), n_requests);
        const cudaError_t er =
            out_bf16 ? mg_launch(gated_recurrence_ranges_kernel<bf16>, rgrid, dim3(32 * RANGE_WARPS), 0, s, true, pre, ld, z_off,
                                 u_off, g_off, req_q_start, req_q_len, req_ctx_before, req_state_slot, state, state_stride,
                                 (bf16*)out, width, n_slots, n_tokens)
                     : mg_launch(gated_recurrence_ranges_kernel<float>, rgrid, dim3(32 * RANGE_WARPS), 0, s, true, pre, ld, z_off,
                                 u_off, g_off, req_q_start, req_q_len, req_ctx_before, req_state_slot, state, state_stride,
                                 (float*)out, width, n_slots, n_tokens);
        if (er != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "gated recurrence (ranges): %s", cudaGetErrorString(er));
        return MG_OK;
    }
    const dim3 grid(ceil_div(width, THREADS), n_requests);
    const cudaError_t e =
        out_bf16 ? mg_launch(gated_recurrence_kernel<bf16>, grid, dim3(THREADS), 0, s, true, pre, ld, z_off, u_off, g_off,
                             req_q_start, req_q_len, req_ctx_before, req_state_slot, state, state_stride, (bf16*)out, width,
                             n_slots, n_tokens)
                 : mg_launch(gated_recurrence_kernel<float>, grid, dim3(THREADS), 0, s, true, pre, ld, z_off, u_off, g_off,
                             req_q_start, req_q_len, req_ctx_before, req_state_slot, state, state_stride, (float*)out, width,
                             n_slots, n_tokens);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "gated recurrence: %s", cudaGetErrorString(e));
    return MG_OK;
}

// x: [n_tokens, width] (bfloat16 if is_bf16 else 32-bit); mu: [n_mixes, width] 32-bit; state: 32-bit slots whose
// first `width` numbers are the request's last input; out: [n_mixes, n_tokens, width] in x's type.
MG_API int mg_token_shift_mix(const void* x, const float* mu, const int* token_request, const int* positions,
                              const int* req_q_start, const int* req_ctx_before, const int* req_state_slot,
                              const float* state, long long state_stride, void* out, int n_tokens, int width, int n_mixes,
                              int n_requests, int n_slots, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && width <= 65535 * THREADS && n_mixes > 0 && n_slots > 0 && state_stride >= width,
               "token shift: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = is_bf16 ? 8 : 4;
    if (width % vec == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 && ((size_t)n_tokens * width) % vec == 0) {
        const dim3 vgrid(n_tokens, ceil_div(width / vec, THREADS));
        const cudaError_t ev =
            is_bf16 ? mg_launch(token_shift_mix_vec_kernel<bf16>, vgrid, dim3(THREADS), 0, s, true, (const bf16*)x, mu,
                                token_request, positions, req_q_start, req_ctx_before, req_state_slot, state, state_stride,
                                (bf16*)out, width, n_mixes, n_tokens, n_requests, n_slots)
                    : mg_launch(token_shift_mix_vec_kernel<float>, vgrid, dim3(THREADS), 0, s, true, (const float*)x, mu,
                                token_request, positions, req_q_start, req_ctx_before, req_state_slot, state, state_stride,
                                (float*)out, width, n_mixes, n_tokens, n_requests, n_slots);
        if (ev != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "token shift: %s", cudaGetErrorString(ev));
        return MG_OK;
    }
    const dim3 grid(n_tokens, ceil_div(width, THREADS));
    const cudaError_t e =
        is_bf16 ? mg_launch(token_shift_mix_kernel<bf16>, grid, dim3(THREADS), 0, s, true, (const bf16*)x, mu, token_request,
                            positions, req_q_start, req_ctx_before, req_state_slot, state, state_stride, (bf16*)out, width,
                            n_mixes, n_tokens, n_requests, n_slots)
                : mg_launch(token_shift_mix_kernel<float>, grid, dim3(THREADS), 0, s, true, (const float*)x, mu,
                            token_request, positions, req_q_start, req_ctx_before, req_state_slot, state, state_stride,
                            (float*)out, width, n_mixes, n_tokens, n_requests, n_slots);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "token shift: %s", cudaGetErrorString(e));
    return MG_OK;
}
