// One small matrix per head, applied to every token's slice of that head:
//
//   out[n, h, j] = sum_i x[n, h, i] * W_h[j, i]      (rows_are_inputs = 0: W is [H * J, I], a head's rows are its outputs)
//   out[n, h, j] = sum_i x[n, h, i] * W_h[i, j]      (rows_are_inputs = 1: W is [H * I, J], a head's rows are its inputs)
//
// optionally times the logistic function of a gate value per output.  An attention whose keys and values are
// made from a small latent per token uses both forms: queries are carried into the latent's space with the
// transposed key matrix of their head (so that scores are taken against the cached latents themselves), and the
// heads' weighted latents are carried to value space with the value matrix of their head.
//
// Tiles of 32 tokens x 64 outputs per CTA, the sum over i in steps of 32 through shared memory, 32-bit
// accumulation in rising order of i whatever the batch.  x, W, the gate and out are bfloat16 or 32-bit alike.
#include "common.cuh"

namespace {

constexpr int TOK = 32, OUT = 64, KC = 32, THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
head_linear_kernel(const T* __restrict__ x, int x_ld, int x_off, int x_head, const T* __restrict__ w, int rows_are_inputs,
                   const T* __restrict__ gate, int gate_ld, T* __restrict__ out, int out_ld, int out_off, int out_head,
                   int n_tokens, int I, int J) {
    __shared__ float xs[TOK][KC + 1];
    __shared__ float ws[KC][OUT + 1];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, h = blockIdx.y;
    const int n0 = blockIdx.x * TOK, j0 = blockIdx.z * OUT;
    const int jl = tid % OUT, tg = tid / OUT;              // this thread: output j0 + jl of tokens tg * 8 .. + 8
    float acc[TOK / 4];
#pragma unroll
    for (int u = 0; u < TOK / 4; ++u) acc[u] = 0.f;
    const T* wh = w + (size_t)h * I * J;
    for (int i0 = 0; i0 < I; i0 += KC) {
        __syncthreads();
        for (int idx = tid; idx < TOK * KC; idx += THREADS) {
            const int t = idx / KC, i = idx - t * KC;
            float v = 0.f;
            if (n0 + t < n_tokens && i0 + i < I) v = to_float(x[(size_t)(n0 + t) * x_ld + x_off + (size_t)h * x_head + i0 + i]);
            xs[t][i] = v;
        }
        if (rows_are_inputs) {
            for (int idx = tid; idx < KC * OUT; idx += THREADS) {
                const int i = idx / OUT, j = idx - i * OUT;
                ws[i][j] = (i0 + i < I && j0 + j < J) ? to_float(wh[(size_t)(i0 + i) * J + j0 + j]) : 0.f;
            }
        } else {
            for (int idx = tid; idx < KC * OUT; idx += THREADS) {
                const int j = idx / KC, i = idx - j * KC;
                ws[i][j] = (i0 + i < I && j0 + j < J) ? to_float(wh[(size_t)(j0 + j) * I + i0 + i]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int i = 0; i < KC; ++i) {
            const float wv = ws[i][jl];
#pragma unroll
            for (int u = 0; u < TOK / 4; ++u) acc[u] = fmaf(xs[tg * (TOK / 4) + u][i], wv, acc[u]);
        }
    }
    if (j0 + jl >= J) return;
#pragma unroll
    for (int u = 0; u < TOK / 4; ++u) {
        const int n = n0 + tg * (TOK / 4) + u;
        if (n >= n_tokens) continue;
        float v = acc[u];
        if (gate) v *= 1.0f / (1.0f + expf(-to_float(gate[(size_t)n * gate_ld + (size_t)h * J + j0 + jl])));
        out[(size_t)n * out_ld + out_off + (size_t)h * out_head + j0 + jl] = from_float<T>(v);
    }
}

}  // namespace

// x: rows of x_ld elements, head h's I inputs from column x_off + h * x_head; w: [n_head * J, I] or, if
// rows_are_inputs, [n_head * I, J]; gate: rows of gate_ld elements whose first n_head * J are gate values, or
// null; out: rows of out_ld elements, head h's J outputs from column out_off + h * out_head.
MG_API int mg_head_linear(const void* x, int x_ld, int x_off, int x_head, const void* w, int rows_are_inputs,
                          const void* gate, int gate_ld, void* out, int out_ld, int out_off, int out_head, int n_tokens,
                          int n_head, int I, int J, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && I > 0 && J > 0, "head_linear: bad sizes");
    MG_REQUIRE(x_off >= 0 && x_head >= I && x_off + (long long)(n_head - 1) * x_head + I <= x_ld &&
                   out_off >= 0 && out_head >= J && out_off + (long long)(n_head - 1) * out_head + J <= out_ld &&
                   (gate == nullptr || gate_ld >= n_head * J),
               "head_linear: heads outside the rows");
    const dim3 grid(ceil_div(n_tokens, TOK), n_head, ceil_div(J, OUT)), block(THREADS);
    MG_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "head_linear: too many heads or outputs");
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t e =
        is_bf16 ? mg_launch(head_linear_kernel<bf16>, grid, block, 0, s, true, (const bf16*)x, x_ld, x_off, x_head,
                            (const bf16*)w, rows_are_inputs, (const bf16*)gate, gate_ld, (bf16*)out, out_ld, out_off,
                            out_head, n_tokens, I, J)
                : mg_launch(head_linear_kernel<float>, grid, block, 0, s, true, (const float*)x, x_ld, x_off, x_head,
                            (const float*)w, rows_are_inputs, (const float*)gate, gate_ld, (float*)out, out_ld, out_off,
                            out_head, n_tokens, I, J);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "head_linear: %s", cudaGetErrorString(e));
    return MG_OK;
}
