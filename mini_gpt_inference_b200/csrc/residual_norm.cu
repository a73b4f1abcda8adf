// What a layer with a norm on both sides of each sublayer, a loop over layers with an additive re-entry, and a
// per-layer token input add to the 32-bit residual stream; all sums and statistics 32-bit.
//
// rmsnorm_add:  x += (y / sqrt(mean(y^2) + eps)) * (offset + w),  y = sa * a [+ sb * b]   (one warp a row; the
//               sublayer's output a, or the weighted sum of two sublayers that ran side by side)
// add_rows:     x += [e] + v    (e: rows like x, or none; v: one row for all tokens)
// scaled_sum:   x += sa * a + sb * b
// softcap:      x <- cap * tanh(x / cap)
// token_gate:   out[t, j] = gelu_tanh(g[t, j]) * table[token_t, off + j]   (a slice of a second embedding table as a
//               gate's other factor; tokens that the step before sampled are taken from its ids, as in the embedding)
// cast_rows:    32-bit rows in the compute type, optionally through tanh
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(residual_norm)

namespace {

constexpr int NORM_WARPS = 4;

__global__ void __launch_bounds__(32 * NORM_WARPS)
rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ a, float sa, const float* __restrict__ b, float sb,
                   const float* __restrict__ w, int rows, int width, float eps, float offset) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* ar = a + (size_t)row * width;
    const float* br = b ? b + (size_t)row * width : nullptr;
    float sq = 0.f;
    for (int c = lane; c < width; c += 32) {
        const float y = br ? fmaf(sb, br[c], sa * ar[c]) : sa * ar[c];
        sq = fmaf(y, y, sq);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    float* xr = x + (size_t)row * width;
    for (int c = lane; c < width; c += 32) {
        const float y = br ? fmaf(sb, br[c], sa * ar[c]) : sa * ar[c];
        xr[c] += y * rstd * (offset + w[c]);
    }
}

__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ e, const float* __restrict__ v,
                                long long n, int width) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float y = x[i] + v[i % width];
    if (e) y += e[i];
    x[i] = y;
}

__global__ void scaled_sum_kernel(float* __restrict__ x, const float* __restrict__ a, float sa,
                                  const float* __restrict__ b, float sb, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += fmaf(sb, b[i], sa * a[i]);
}

__global__ void softcap_kernel(float* x, long long n, float cap) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long n, int use_tanh) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<T>(use_tanh ? tanhf(x[i]) : x[i]);
}

template <typename TW, typename T>
__global__ void token_gate_kernel(const float* __restrict__ g, const int* __restrict__ ids, const int* __restrict__ pos,
                                  const int* __restrict__ source, const int* __restrict__ previous,
                                  const TW* __restrict__ table, int table_ld, int off, T* __restrict__ out, int dim,
                                  int vocab, int n_previous) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    T* orow = out + (size_t)n * dim;
    if (pos[n] < 0) {
        for (int j = threadIdx.x; j < dim; j += blockDim.x) orow[j] = from_float<T>(0.f);
        return;
    }
    int id = ids[n];
    if (source != nullptr) {
        const int src = source[n];
        if (src >= 0 && MG_GUARDED(residual_norm, MG_GUARD_SOURCE, src, n_previous)) id = previous[src];
    }
    if (!MG_GUARDED(residual_norm, MG_GUARD_TOKEN, id, vocab)) id = 0;
    const TW* trow = table + (size_t)id * table_ld + off;
    const float* grow = g + (size_t)n * dim;
    for (int j = threadIdx.x; j < dim; j += blockDim.x) {
        const float z = grow[j];
        const float act = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
        orow[j] = from_float<T>(act * to_float(trow[j]));
    }
}

}  // namespace

// x: [rows, width] 32-bit, in place; a (and b, or null): [rows, width] 32-bit; w: [width] 32-bit.
MG_API int mg_rmsnorm_add(float* x, const float* a, float sa, const float* b, float sb, const float* w, int rows,
                          int width, float eps, float offset, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && width > 0 && x && a && w, "rmsnorm_add: bad sizes");
    const cudaError_t e = mg_launch(rmsnorm_add_kernel, dim3(ceil_div(rows, NORM_WARPS)), dim3(32 * NORM_WARPS), 0,
                                    (cudaStream_t)stream, true, x, a, sa, b, sb, w, rows, width, eps, offset);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "rmsnorm_add: %s", cudaGetErrorString(e));
    return MG_OK;
}

// x: [n / width, width] 32-bit, in place; e: the same shape or null; v: [width] 32-bit.
MG_API int mg_add_rows(float* x, const float* e, const float* v, long long n, int width, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && n < (1ll << 40) && width > 0 && n % width == 0 && v, "add_rows: bad sizes");
    const cudaError_t err = mg_launch(add_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                      (cudaStream_t)stream, true, x, e, v, n, width);
    if (err != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "add_rows: %s", cudaGetErrorString(err));
    return MG_OK;
}

MG_API int mg_scaled_sum(float* x, const float* a, float sa, const float* b, float sb, long long n, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && n < (1ll << 40) && a && b, "scaled_sum: bad sizes");
    const cudaError_t e = mg_launch(scaled_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                    (cudaStream_t)stream, true, x, a, sa, b, sb, n);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "scaled_sum: %s", cudaGetErrorString(e));
    return MG_OK;
}

MG_API int mg_softcap(float* x, long long n, float cap, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && n < (1ll << 40) && cap > 0.f, "softcap: bad size or cap");
    const cudaError_t e = mg_launch(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                                    true, x, n, cap);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "softcap: %s", cudaGetErrorString(e));
    return MG_OK;
}

// out[i] = x[i], or tanh(x[i]) if use_tanh, in bfloat16 (out_bf16) or 32-bit (out may then be x itself).
MG_API int mg_cast_rows(const float* x, void* out, long long n, int use_tanh, int out_bf16, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && n < (1ll << 40), "cast: bad size");
    const dim3 grid((unsigned)((n + 255) / 256));
    const cudaError_t e =
        out_bf16 ? mg_launch(cast_rows_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, true, x, (bf16*)out, n, use_tanh)
                 : mg_launch(cast_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, true, x, (float*)out, n, use_tanh);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "cast: %s", cudaGetErrorString(e));
    return MG_OK;
}

// g: [n_tokens, dim] 32-bit; table: [vocab, table_ld] (bfloat16 if table_bf16 else 32-bit), of which columns
// off .. off + dim - 1 are read; out: [n_tokens, dim] (bfloat16 if out_bf16 else 32-bit).  source / previous as in
// mg_embed; n_previous: ids that `previous` holds.
MG_API int mg_token_gate(const float* g, const int* ids, const int* pos, const int* source, const int* previous,
                         const void* table, int table_ld, int off, void* out, int n_tokens, int dim, int vocab,
                         int n_previous, int table_bf16, int out_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && dim > 0 && vocab > 0 && off >= 0 && off + dim <= table_ld, "token_gate: bad sizes");
    MG_REQUIRE(source == nullptr || previous != nullptr, "token_gate: token sources without the ids they point to");
    MG_REQUIRE(table_bf16 == out_bf16, "token_gate: the table and the output share a type");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = dim >= 128 ? 128 : dim >= 64 ? 64 : 32;
    const cudaError_t e =
        out_bf16 ? mg_launch(token_gate_kernel<bf16, bf16>, dim3(n_tokens), dim3(threads), 0, s, true, g, ids, pos, source,
                             previous, (const bf16*)table, table_ld, off, (bf16*)out, dim, vocab, n_previous)
                 : mg_launch(token_gate_kernel<float, float>, dim3(n_tokens), dim3(threads), 0, s, true, g, ids, pos, source,
                             previous, (const float*)table, table_ld, off, (float*)out, dim, vocab, n_previous);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "token_gate: %s", cudaGetErrorString(e));
    return MG_OK;
}
