// What a state-space mixer does around its scan, besides the projections.
//
// causal_conv_silu: a short causal convolution per channel over a request's tokens, then silu:
//   y_t[c] = silu(bias[c] + sum_j taps[c][j] * x_(t - (n - 1) + j)[c]),   j = 0 .. n - 1 (the last tap weighs token t)
// with zeros before the sequence's start.  The n - 1 inputs before a step's first token come from the request's
// state slot ([n - 1][channels] 32-bit, oldest first); conv_state_update then leaves the last n - 1 inputs of the
// sequence there for the next step (a kernel of its own: every token of the step may still read the old ones).
//
// gated_group_norm: out = rms_norm_in_parts(o * silu(z)) * gain: the scan's 32-bit output times silu of the gate
// columns, the row cut into `parts` equal parts, each divided by its own root mean square (eps inside the root).
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(short_conv)

namespace {

constexpr int THREADS = 128;
constexpr int MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(THREADS)
causal_conv_silu_kernel(const T* __restrict__ x, int ld, int x_off, const float* __restrict__ taps,
                        const float* __restrict__ bias, const int* __restrict__ token_request,
                        const int* __restrict__ positions, const int* __restrict__ req_q_start,
                        const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                        const float* __restrict__ state, long long state_stride, T* __restrict__ out, int channels,
                        int n_taps, int n_requests, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.y, c = blockIdx.x * THREADS + threadIdx.x;
    if (c >= channels || positions[token] < 0) return;
    int r = token_request[token];
    if (!MG_GUARDED(short_conv, MG_GUARD_REQUEST, r, n_requests)) return;
    const int start = req_q_start[r], local = token - start;
    int slot = req_state_slot[r];
    if (!MG_GUARDED(short_conv, MG_GUARD_ROW, slot, n_slots)) return;
    const bool fresh = req_ctx_before[r] == 0;
    const float* old = state + (size_t)slot * state_stride;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < n_taps; ++j) {
        const int back = local - (n_taps - 1) + j;         // the input's place among the step's tokens of the request
        float v;
        if (back >= 0) v = to_float(x[(size_t)(start + back) * ld + x_off + c]);
        else v = fresh ? 0.f : old[(size_t)(n_taps - 1 + back) * channels + c];
        acc = fmaf(taps[(size_t)c * n_taps + j], v, acc);
    }
    out[(size_t)token * channels + c] = from_float<T>(acc / (1.0f + expf(-acc)));
}

// Eight neighbouring channels and TT consecutive tokens of the step per thread, 16-byte loads and stores; each
// output's sum runs over the taps in the same rising order as in the kernel above, so both give the same bits.
template <typename T>
__device__ __forceinline__ void load8(float (&v)[8], const T* p);
template <>
__device__ __forceinline__ void load8<float>(float (&v)[8], const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(float (&v)[8], const bf16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        v[2 * u] = __bfloat162float(h[u].x);
        v[2 * u + 1] = __bfloat162float(h[u].y);
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int u = 0; u < 4; ++u) h[u] = __floats2bfloat162_rn(v[2 * u], v[2 * u + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

template <typename T, int TT>
__global__ void __launch_bounds__(THREADS)
causal_conv_silu_vec_kernel(const T* __restrict__ x, int ld, int x_off, const float* __restrict__ taps,
                            const float* __restrict__ bias, const int* __restrict__ token_request,
                            const int* __restrict__ positions, const int* __restrict__ req_q_start,
                            const int* __restrict__ req_ctx_before, const int* __restrict__ req_state_slot,
                            const float* __restrict__ state, long long state_stride, T* __restrict__ out, int channels,
                            int n_taps, int n_requests, int n_slots, int n_tokens) {
    pdl_trigger();
    pdl_wait();
    const int c = (blockIdx.x * THREADS + threadIdx.x) * 8, t0 = blockIdx.y * TT;
    if (c >= channels) return;
    int start[TT], local[TT];
    const float* old[TT];                                  // null: zeros before the sequence's start
    bool live[TT];
    float acc[TT][8];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        const int token = t0 + tt;
        live[tt] = token < n_tokens && positions[token] >= 0;
        start[tt] = local[tt] = 0;
        old[tt] = nullptr;
        if (live[tt]) {
            int r = token_request[token];
            if (!MG_GUARDED(short_conv, MG_GUARD_REQUEST, r, n_requests)) { live[tt] = false; continue; }
            int slot = req_state_slot[r];
            if (!MG_GUARDED(short_conv, MG_GUARD_ROW, slot, n_slots)) { live[tt] = false; continue; }
            start[tt] = req_q_start[r];
            local[tt] = token - start[tt];
            if (req_ctx_before[r] != 0) old[tt] = state + (size_t)slot * state_stride;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[tt][u] = bias ? bias[c + u] : 0.f;
    }
    for (int j = 0; j < n_taps; ++j) {
        float w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = taps[(size_t)(c + u) * n_taps + j];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            if (!live[tt]) continue;
            const int back = local[tt] - (n_taps - 1) + j;
            float v[8];
            if (back >= 0) load8<T>(v, x + (size_t)(start[tt] + back) * ld + x_off + c);
            else if (old[tt]) load8<float>(v, old[tt] + (size_t)(n_taps - 1 + back) * channels + c);
            else {
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[tt][u] = fmaf(w[u], v[u], acc[tt][u]);
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
        if (!live[tt]) continue;
#pragma unroll
        for (int u = 0; u < 8; ++u)                        // (bfloat16 results: the fast exponential and division are far
            acc[tt][u] = sizeof(T) == 2 ? __fdividef(acc[tt][u], 1.0f + __expf(-acc[tt][u]))   //  inside their rounding)
                                        : acc[tt][u] / (1.0f + expf(-acc[tt][u]));
        store8(out + (size_t)(t0 + tt) * channels + c, acc[tt]);
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
conv_state_update_kernel(const T* __restrict__ x, int ld, int x_off, const int* __restrict__ req_q_start,
                         const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_before,
                         const int* __restrict__ req_state_slot, float* __restrict__ state, long long state_stride,
                         int channels, int n_taps, int n_slots) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.y, c = blockIdx.x * THREADS + threadIdx.x;
    const int q_len = req_q_len[r];
    if (c >= channels || q_len <= 0) return;
    int slot = req_state_slot[r];
    if (!MG_GUARDED(short_conv, MG_GUARD_ROW, slot, n_slots)) return;
    const bool fresh = req_ctx_before[r] == 0;
    const int start = req_q_start[r], keep = n_taps - 1;
    float* mine = state + (size_t)slot * state_stride;
    float next[MAX_TAPS - 1];
#pragma unroll
    for (int s = 0; s < MAX_TAPS - 1; ++s) {
        if (s >= keep) break;
        const int back = q_len - keep + s;                 // among the step's tokens; negative: an older input
        if (back >= 0) next[s] = to_float(x[(size_t)(start + back) * ld + x_off + c]);
        else next[s] = fresh ? 0.f : mine[(size_t)(keep + back) * channels + c];
    }
#pragma unroll
    for (int s = 0; s < MAX_TAPS - 1; ++s) {
        if (s >= keep) break;
        mine[(size_t)s * channels + c] = next[s];
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
gated_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ z, int z_ld, const float* __restrict__ gain,
                        const int* __restrict__ positions, T* __restrict__ out, int width, int parts, float eps) {
    __shared__ float red[THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, part = blockIdx.y, tid = threadIdx.x;
    const int size = width / parts, first = part * size;
    T* orow = out + (size_t)token * width + first;
    if (positions != nullptr && positions[token] < 0) {
        for (int i = tid; i < size; i += THREADS) orow[i] = from_float<T>(0.f);
        return;
    }
    const float* src = o + (size_t)token * width + first;
    const T* gate = z + (size_t)token * z_ld + first;
    float sq = 0.f;
    for (int i = tid; i < size; i += THREADS) {
        const float g = to_float(gate[i]);
        const float v = src[i] * (g / (1.0f + expf(-g)));
        sq = fmaf(v, v, sq);
    }
    sq = warp_sum(sq);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) total += red[w];
    const float rstd = 1.0f / sqrtf(total / (float)size + eps);
    for (int i = tid; i < size; i += THREADS) {
        const float g = to_float(gate[i]);
        orow[i] = from_float<T>(src[i] * (g / (1.0f + expf(-g))) * rstd * gain[first + i]);
    }
}

}  // namespace

// x: rows of ld elements whose `channels` columns from x_off are the convolution's inputs; taps: [channels, n_taps]
// 32-bit (the last column weighs the current token); bias: [channels] 32-bit or null; token_request, positions:
// [n_tokens]; req_*: [n_requests]; state: [n_slots, state_stride] 32-bit, the convolution's part of a slot first
// ((n_taps - 1) x channels numbers); out: [n_tokens, channels].
MG_API int mg_causal_conv_silu(const void* x, int ld, int x_off, const float* taps, const float* bias,
                               const int* token_request, const int* positions, const int* req_q_start,
                               const int* req_ctx_before, const int* req_state_slot, const float* state,
                               long long state_stride, void* out, int n_tokens, int channels, int n_taps, int n_requests,
                               int n_slots, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && channels > 0 && n_taps > 0 && n_taps <= MAX_TAPS && x_off >= 0 && x_off + channels <= ld,
               "causal_conv: bad sizes (1..%d taps)", MAX_TAPS);
    MG_REQUIRE(state_stride >= (long long)(n_taps - 1) * channels && n_tokens <= 65535 * 1024, "causal_conv: the state slots are too small");
    const dim3 grid(ceil_div(channels, THREADS), n_tokens), block(THREADS);
    MG_REQUIRE(grid.y <= 65535u * 32768u, "causal_conv: too many tokens");
    cudaStream_t s = (cudaStream_t)stream;
    if (channels % 8 == 0 && ld % 8 == 0 && x_off % 8 == 0 && state_stride % 4 == 0 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)out % 16 == 0 && (uintptr_t)state % 16 == 0 && n_tokens <= 65535) {
        const bool many = n_tokens > 64;                   // few tokens: one per thread, for more threads
        const dim3 g(ceil_div(channels / 8, THREADS), many ? ceil_div(n_tokens, 4) : n_tokens);
#define MG_CONV_VEC(T, TT)                                                                                              \
    mg_launch(causal_conv_silu_vec_kernel<T, TT>, g, block, 0, s, true, (const T*)x, ld, x_off, taps, bias, token_request, \
              positions, req_q_start, req_ctx_before, req_state_slot, state, state_stride, (T*)out, channels, n_taps,     \
              n_requests, n_slots, n_tokens)
        const cudaError_t e = is_bf16 ? (many ? MG_CONV_VEC(bf16, 4) : MG_CONV_VEC(bf16, 1))
                                      : (many ? MG_CONV_VEC(float, 4) : MG_CONV_VEC(float, 1));
#undef MG_CONV_VEC
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "causal_conv: %s", cudaGetErrorString(e));
        return MG_OK;
    }
    // (the grid's second dimension takes 65,535 rows: longer steps run in slices)
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        const dim3 g(grid.x, nt);
        const cudaError_t e =
            is_bf16 ? mg_launch(causal_conv_silu_kernel<bf16>, g, block, 0, s, true, (const bf16*)x, ld, x_off, taps, bias,
                                token_request + t0, positions + t0, req_q_start, req_ctx_before, req_state_slot, state,
                                state_stride, (bf16*)out + (size_t)t0 * channels, channels, n_taps, n_requests, n_slots)
                    : mg_launch(causal_conv_silu_kernel<float>, g, block, 0, s, true, (const float*)x, ld, x_off, taps, bias,
                                token_request + t0, positions + t0, req_q_start, req_ctx_before, req_state_slot, state,
                                state_stride, (float*)out + (size_t)t0 * channels, channels, n_taps, n_requests, n_slots);
        if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "causal_conv: %s", cudaGetErrorString(e));
    }
    return MG_OK;
}

// After mg_causal_conv_silu of the same step: the last n_taps - 1 inputs of every request's sequence into its slot.
MG_API int mg_conv_state_update(const void* x, int ld, int x_off, const int* req_q_start, const int* req_q_len,
                                const int* req_ctx_before, const int* req_state_slot, float* state, long long state_stride,
                                int n_requests, int channels, int n_taps, int n_slots, int is_bf16, void* stream) {
    if (n_requests == 0 || n_taps <= 1) return MG_OK;
    MG_REQUIRE(n_requests > 0 && n_requests <= 65535 && channels > 0 && n_taps <= MAX_TAPS && x_off >= 0 && x_off + channels <= ld,
               "conv_state_update: bad sizes");
    MG_REQUIRE(state_stride >= (long long)(n_taps - 1) * channels, "conv_state_update: the state slots are too small");
    const dim3 grid(ceil_div(channels, THREADS), n_requests), block(THREADS);
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t e =
        is_bf16 ? mg_launch(conv_state_update_kernel<bf16>, grid, block, 0, s, true, (const bf16*)x, ld, x_off, req_q_start,
                            req_q_len, req_ctx_before, req_state_slot, state, state_stride, channels, n_taps, n_slots)
                : mg_launch(conv_state_update_kernel<float>, grid, block, 0, s, true, (const float*)x, ld, x_off, req_q_start,
                            req_q_len, req_ctx_before, req_state_slot, state, state_stride, channels, n_taps, n_slots);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "conv_state_update: %s", cudaGetErrorString(e));
    return MG_OK;
}

// o: [n_tokens, width] 32-bit; z: rows of z_ld elements whose first `width` are the gate's pre-activations; gain:
// [width] 32-bit; positions: [n_tokens] or null (rows with a negative one become zeros); out: [n_tokens, width] in
// z's type.  width must be a multiple of parts.
MG_API int mg_gated_group_norm(const float* o, const void* z, int z_ld, const float* gain, const int* positions, void* out,
                               int n_tokens, int width, int parts, float eps, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && width > 0 && parts > 0 && width % parts == 0 && parts <= 65535 && z_ld >= width,
               "gated_group_norm: bad sizes");
    const dim3 grid(n_tokens, parts), block(THREADS);
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t e =
        is_bf16 ? mg_launch(gated_group_norm_kernel<bf16>, grid, block, 0, s, true, o, (const bf16*)z, z_ld, gain, positions,
                            (bf16*)out, width, parts, eps)
                : mg_launch(gated_group_norm_kernel<float>, grid, block, 0, s, true, o, (const float*)z, z_ld, gain, positions,
                            (float*)out, width, parts, eps);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "gated_group_norm: %s", cudaGetErrorString(e));
    return MG_OK;
}
