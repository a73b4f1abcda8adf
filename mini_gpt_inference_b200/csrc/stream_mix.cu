// Several residual streams side by side ("hyper-connections"): instead of one stream x there are S copies
// x_0 .. x_(S-1), stored [S][tokens][width] in 32-bit.  A sublayer reads one mixture of them and its
// output is written back into every stream while the streams are mixed among themselves:
//
//   read:    u = sum_s a[s] x_s
//   write:   x'_t = sum_s M[s][t] x_s + b[t] y          (all t at once, from the old streams)
//   write + read:  the write, and u' = sum_t a'[t] x'_t for the sublayer that follows, in one pass
//   sum:     x = sum_s x_s                               (what the model's final norm reads)
//   spread:  x_s = x for every s                         (the embedding's output, copied into every stream)
//
// Everything is 32-bit and element-wise, every sum runs over s in rising order, so an element's value does
// not depend on the batch it is computed in.  `read` can also fill a second buffer with zeros: the sublayer
// adds its output into that buffer with the projections' residual epilogue, and `write` takes it as y.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;
constexpr int THREADS = 256;

__device__ __forceinline__ float4 fma4(float w, float4 x, float4 acc) {
    return make_float4(fmaf(w, x.x, acc.x), fmaf(w, x.y, acc.y), fmaf(w, x.z, acc.z), fmaf(w, x.w, acc.w));
}

// weights live in device memory (they are the model's tensors); every thread reads the few it needs
template <int VEC>
__global__ void __launch_bounds__(THREADS)
streams_read_kernel(const float* __restrict__ x, const float* __restrict__ a, float* __restrict__ u,
                    float* __restrict__ zero, int S, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = ((long long)blockIdx.x * THREADS + threadIdx.x) * VEC;
    if (i >= n) return;
    if (VEC == 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < S; ++s) acc = fma4(a[s], *reinterpret_cast<const float4*>(x + (size_t)s * n + i), acc);
        *reinterpret_cast<float4*>(u + i) = acc;
        if (zero) *reinterpret_cast<float4*>(zero + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        float acc = 0.f;
        for (int s = 0; s < S; ++s) acc = fmaf(a[s], x[(size_t)s * n + i], acc);
        u[i] = acc;
        if (zero) zero[i] = 0.f;
    }
}

template <int VEC>
__global__ void __launch_bounds__(THREADS)
streams_write_kernel(float* __restrict__ x, const float* __restrict__ mix, const float* __restrict__ b,
                     const float* __restrict__ y, const float* __restrict__ a_next, float* __restrict__ u_next,
                     float* __restrict__ zero, int S, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = ((long long)blockIdx.x * THREADS + threadIdx.x) * VEC;
    if (i >= n) return;
    if (VEC == 4) {
        float4 old[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) old[s] = *reinterpret_cast<const float4*>(x + (size_t)s * n + i);
        const float4 yv = *reinterpret_cast<const float4*>(y + i);
        float4 un = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
            if (t >= S) break;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) acc = fma4(mix[s * S + t], old[s], acc);
            acc = fma4(b[t], yv, acc);
            *reinterpret_cast<float4*>(x + (size_t)t * n + i) = acc;
            if (u_next) un = fma4(a_next[t], acc, un);
        }
        if (u_next) *reinterpret_cast<float4*>(u_next + i) = un;
        if (zero) *reinterpret_cast<float4*>(zero + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        float old[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) old[s] = x[(size_t)s * n + i];
        const float yv = y[i];
        float un = 0.f;
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
            if (t >= S) break;
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) acc = fmaf(mix[s * S + t], old[s], acc);
            acc = fmaf(b[t], yv, acc);
            x[(size_t)t * n + i] = acc;
            if (u_next) un = fmaf(a_next[t], acc, un);
        }
        if (u_next) u_next[i] = un;
        if (zero) zero[i] = 0.f;
    }
}

template <int VEC>
__global__ void __launch_bounds__(THREADS)
streams_spread_kernel(const float* __restrict__ src, float* __restrict__ x, int S, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = ((long long)blockIdx.x * THREADS + threadIdx.x) * VEC;
    if (i >= n) return;
    if (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        for (int s = 0; s < S; ++s) *reinterpret_cast<float4*>(x + (size_t)s * n + i) = v;
    } else {
        const float v = src[i];
        for (int s = 0; s < S; ++s) x[(size_t)s * n + i] = v;
    }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace

// x: [S, n] 32-bit (n = tokens * width); a: [S] on the device; u: [n]; zero: [n] or null (filled with zeros).
MG_API int mg_streams_read(const float* x, const float* a, float* u, float* zero, int S, long long n, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(S > 0 && S <= MAX_STREAMS && n > 0, "streams: 1..%d streams", MAX_STREAMS);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && aligned16(x) && aligned16(u) && (zero == nullptr || aligned16(zero));
    const long long items = vec ? n / 4 : n;
    const dim3 grid((unsigned)((items + THREADS - 1) / THREADS)), block(THREADS);
    const cudaError_t e = vec ? mg_launch(streams_read_kernel<4>, grid, block, 0, s, true, x, a, u, zero, S, n)
                              : mg_launch(streams_read_kernel<1>, grid, block, 0, s, true, x, a, u, zero, S, n);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "streams (read): %s", cudaGetErrorString(e));
    return MG_OK;
}

// x: [S, n] updated in place; mix: [S, S] indexed [from][to]; b: [S]; y: [n].  With a_next and u_next (both or
// neither): u_next = sum_t a_next[t] x'_t as well; zero: [n] or null, filled with zeros
// (another buffer than y).
MG_API int mg_streams_write(float* x, const float* mix, const float* b, const float* y, const float* a_next,
                            float* u_next, float* zero, int S, long long n, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(S > 0 && S <= MAX_STREAMS && n > 0, "streams: 1..%d streams", MAX_STREAMS);
    MG_REQUIRE((a_next == nullptr) == (u_next == nullptr), "streams: the next read wants its weights and its room");
    MG_REQUIRE(u_next != y && (zero == nullptr || zero != y), "streams: the output of this sublayer is only read");
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && aligned16(x) && aligned16(y) && (u_next == nullptr || aligned16(u_next)) &&
                     (zero == nullptr || aligned16(zero));
    const long long items = vec ? n / 4 : n;
    const dim3 grid((unsigned)((items + THREADS - 1) / THREADS)), block(THREADS);
    const cudaError_t e =
        vec ? mg_launch(streams_write_kernel<4>, grid, block, 0, s, true, x, mix, b, y, a_next, u_next, zero, S, n)
            : mg_launch(streams_write_kernel<1>, grid, block, 0, s, true, x, mix, b, y, a_next, u_next, zero, S, n);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "streams (write): %s", cudaGetErrorString(e));
    return MG_OK;
}

// x[s] = src for every s.
MG_API int mg_streams_spread(const float* src, float* x, int S, long long n, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(S > 0 && S <= MAX_STREAMS && n > 0, "streams: 1..%d streams", MAX_STREAMS);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && aligned16(x) && aligned16(src);
    const long long items = vec ? n / 4 : n;
    const dim3 grid((unsigned)((items + THREADS - 1) / THREADS)), block(THREADS);
    const cudaError_t e = vec ? mg_launch(streams_spread_kernel<4>, grid, block, 0, s, true, src, x, S, n)
                              : mg_launch(streams_spread_kernel<1>, grid, block, 0, s, true, src, x, S, n);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "streams (spread): %s", cudaGetErrorString(e));
    return MG_OK;
}
