// What a layer with a norm on both sides of each sublayer, a loop over layers with an additive re-entry, and a
// per-layer token input add to the 32-bit residual stream; all sums and statistics 32-bit.
//
// rmsnorm_add:  x += (y / sqrt(mean(y^2) + eps)) * (offset + w),  y = sa * a [+ sb * b]   (one warp a row; the
//               sublayer's output a, or the weighted sum of two sublayers that ran side by side).  With `clear` the
//               inputs are left as zeros: the buffer a sublayer added its output into serves the next sublayer as it is
// add_rows:     x += [e] + v    (e: rows like x, or none; v: one row for all tokens)
// scaled_sum:   x += sa * a + sb * b   (with `clear`, a and b are left as zeros)
// softcap:      x <- cap * tanh(x / cap)
// token_gate:   out[t, j] = gelu_tanh(g[t, j]) * table[token_t, off + j]   (a slice of a second embedding table as a
//               gate's other factor; tokens that the step before sampled are taken from its ids, as in the embedding)
// cast_rows:    32-bit rows in the compute type, optionally through tanh
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(residual_norm)

namespace {

constexpr int NORM_WARPS = 4;
constexpr int ROW_THREADS = 256;   // threads of the CTA that owns a row in the vector form
constexpr int MAX_ROW_VECS = 8;    // most float4 a thread holds: rows of up to 256 * 8 * 4 = 8,192 numbers

// The general form: one warp a row, two passes over the row (any width).
__global__ void __launch_bounds__(32 * NORM_WARPS)
rmsnorm_add_kernel(float* __restrict__ x, float* __restrict__ a, float sa, float* __restrict__ b, float sb,
                   const float* __restrict__ w, int rows, int width, float eps, float offset, int clear) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* ar = a + (size_t)row * width;
    float* br = b ? b + (size_t)row * width : nullptr;
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
        if (clear) {
            ar[c] = 0.f;
            if (br) br[c] = 0.f;
        }
    }
}

// The vector form: one CTA a row, the row's numbers asked for at once (16 bytes a load) and held in registers
// between the statistics and the sum, so that a step of few rows is one trip to memory and not a chain of them.
template <int ROW_VECS>       // float4 a thread holds: 1, 2, 4 or 8 (rows of up to 1,024 ... 8,192 numbers)
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_add_vec_kernel(float* __restrict__ x, float* __restrict__ a, float sa, float* __restrict__ b, float sb,
                       const float* __restrict__ w, int width, float eps, float offset, int clear) {
    __shared__ float red[ROW_THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int vecs = width >> 2, tid = threadIdx.x;
    float4* ar = reinterpret_cast<float4*>(a + (size_t)blockIdx.x * width);
    float4* br = b ? reinterpret_cast<float4*>(b + (size_t)blockIdx.x * width) : nullptr;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)blockIdx.x * width);
    const float4* wr = reinterpret_cast<const float4*>(w);
    float4 y[ROW_VECS], xv[ROW_VECS], wv[ROW_VECS];
#pragma unroll
    for (int u = 0; u < ROW_VECS; ++u) {
        const int i = tid + u * ROW_THREADS;
        y[u] = xv[u] = wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < vecs) {
            const float4 av = ar[i];
            y[u] = make_float4(sa * av.x, sa * av.y, sa * av.z, sa * av.w);
            if (br) {
                const float4 bv = br[i];
                y[u] = make_float4(fmaf(sb, bv.x, y[u].x), fmaf(sb, bv.y, y[u].y), fmaf(sb, bv.z, y[u].z), fmaf(sb, bv.w, y[u].w));
            }
            xv[u] = xr[i];
            wv[u] = wr[i];
        }
    }
    float sq = 0.f;
#pragma unroll
    for (int u = 0; u < ROW_VECS; ++u) sq = fmaf(y[u].x, y[u].x, fmaf(y[u].y, y[u].y, fmaf(y[u].z, y[u].z, fmaf(y[u].w, y[u].w, sq))));
    sq = warp_sum(sq);
    if ((tid & 31) == 0) red[tid >> 5] = sq;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < ROW_THREADS / 32; ++k) total += red[k];
    const float rstd = 1.0f / sqrtf(total / (float)width + eps);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < ROW_VECS; ++u) {
        const int i = tid + u * ROW_THREADS;
        if (i < vecs) {
            xr[i] = make_float4(xv[u].x + y[u].x * rstd * (offset + wv[u].x), xv[u].y + y[u].y * rstd * (offset + wv[u].y),
                                xv[u].z + y[u].z * rstd * (offset + wv[u].z), xv[u].w + y[u].w * rstd * (offset + wv[u].w));
            if (clear) {
                ar[i] = zero;
                if (br) br[i] = zero;
            }
        }
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

__global__ void scaled_sum_kernel(float* __restrict__ x, float* __restrict__ a, float sa, float* __restrict__ b, float sb,
                                  long long n, int clear) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    x[i] += fmaf(sb, b[i], sa * a[i]);
    if (clear) a[i] = b[i] = 0.f;
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

// x: [rows, width] 32-bit, in place; a (and b, or null): [rows, width] 32-bit (zeroed if clear); w: [width] 32-bit.
MG_API int mg_rmsnorm_add(float* x, float* a, float sa, float* b, float sb, const float* w, int rows,
                          int width, float eps, float offset, int clear, void* stream) {
    if (rows == 0) return MG_OK;
    MG_REQUIRE(rows > 0 && width > 0 && x && a && w, "rmsnorm_add: bad sizes");
    const bool vec = width % 4 == 0 && width <= ROW_THREADS * MAX_ROW_VECS * 4 && (uintptr_t)x % 16 == 0 && (uintptr_t)a % 16 == 0 &&
                     (uintptr_t)b % 16 == 0 && (uintptr_t)w % 16 == 0;
    const int per_thread = ceil_div(width / 4, ROW_THREADS);
    auto vec_kernel = per_thread <= 1 ? rmsnorm_add_vec_kernel<1> : per_thread <= 2 ? rmsnorm_add_vec_kernel<2>
                    : per_thread <= 4 ? rmsnorm_add_vec_kernel<4> : rmsnorm_add_vec_kernel<8>;
    const cudaError_t e =
        vec ? mg_launch(vec_kernel, dim3(rows), dim3(ROW_THREADS), 0, (cudaStream_t)stream, true, x, a, sa, b, sb, w,
                        width, eps, offset, clear)
            : mg_launch(rmsnorm_add_kernel, dim3(ceil_div(rows, NORM_WARPS)), dim3(32 * NORM_WARPS), 0, (cudaStream_t)stream,
                        true, x, a, sa, b, sb, w, rows, width, eps, offset, clear);
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

MG_API int mg_scaled_sum(float* x, float* a, float sa, float* b, float sb, long long n, int clear, void* stream) {
    if (n == 0) return MG_OK;
    MG_REQUIRE(n > 0 && n < (1ll << 40) && a && b, "scaled_sum: bad sizes");
    const cudaError_t e = mg_launch(scaled_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                    (cudaStream_t)stream, true, x, a, sa, b, sb, n, clear);
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
