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
// (bfloat16 steps take the tensor-core kernel further down where 16-byte loads fit.)
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


// bfloat16 with many tokens: tiles of 128 tokens x 64 outputs per CTA of four warps (32 tokens a warp, so that a
// fragment of the head's matrix serves two products) on the warp-level tensor cores
// (mma.sync m16n8k16, 32-bit accumulation), the sum over i in steps of 64 through shared memory.  A head's matrix is
// read as it lies: rows that are outputs through ldmatrix, rows that are inputs through ldmatrix.trans.  A token's
// result depends on its own row only.
constexpr int MT = 128, MK = 64, MPAD = 8;

__device__ __forceinline__ void hl_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void hl_ldsm(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void hl_ldsm_t(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <int MN>            // outputs per CTA: 64, or 16 for steps of few tokens (more CTAs share the heads' matrices)
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const bf16* __restrict__ x, int x_ld, int x_off, int x_head, const bf16* __restrict__ w,
                       int rows_are_inputs, const bf16* __restrict__ gate, int gate_ld, bf16* __restrict__ out, int out_ld,
                       int out_off, int out_head, int n_tokens, int I, int J) {
    __shared__ __align__(16) bf16 xs[MT][MK + MPAD];
    __shared__ __align__(16) bf16 ws[64][64 + MPAD];       // [j][i], or [i][j] if the rows are inputs
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, h = blockIdx.y;
    const int n0 = blockIdx.x * MT, j0 = blockIdx.z * MN;
    float acc[2][MN / 8][4];
#pragma unroll
    for (int n = 0; n < MN / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][n][e] = acc[1][n][e] = 0.f;
    const bf16* wh = w + (size_t)h * I * J;
    const bf16* xh = x + x_off + (size_t)h * x_head;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i0 = 0; i0 < I; i0 += MK) {
        __syncthreads();
        for (int idx = tid; idx < MT * (MK / 8); idx += 128) {
            const int t = idx >> 3, c = (idx & 7) * 8;
            *reinterpret_cast<uint4*>(&xs[t][c]) =
                (n0 + t < n_tokens && i0 + c < I) ? *reinterpret_cast<const uint4*>(xh + (size_t)(n0 + t) * x_ld + i0 + c) : zero;
        }
        for (int idx = tid; idx < 64 * 8; idx += 128) {
            const int r = idx >> 3, c = (idx & 7) * 8;
            uint4 v = zero;
            if (rows_are_inputs) {
                if (c < MN && i0 + r < I && j0 + c < J) v = *reinterpret_cast<const uint4*>(wh + (size_t)(i0 + r) * J + j0 + c);
            } else {
                if (r < MN && j0 + r < J && i0 + c < I) v = *reinterpret_cast<const uint4*>(wh + (size_t)(j0 + r) * I + i0 + c);
            }
            *reinterpret_cast<uint4*>(&ws[r][c]) = v;
        }
        __syncthreads();
        if (n0 + warp * 32 >= n_tokens) continue;          // a warp without tokens only helps with the loads
#pragma unroll
        for (int kk = 0; kk < MK; kk += 16) {
            uint32_t a0[4], a1[4];
            hl_ldsm(a0, &xs[warp * 32 + (lane & 15)][kk + (lane >> 4) * 8]);
            hl_ldsm(a1, &xs[warp * 32 + 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int n = 0; n < MN / 8; n += 2) {
                uint32_t b[4];
                if (rows_are_inputs) hl_ldsm_t(b, &ws[kk + ((lane >> 3) & 1) * 8 + (lane & 7)][n * 8 + (lane >> 4) * 8]);
                else hl_ldsm(b, &ws[n * 8 + (lane >> 4) * 8 + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
                hl_mma(acc[0][n], a0, b[0], b[1]);
                hl_mma(acc[0][n + 1], a0, b[2], b[3]);
                hl_mma(acc[1][n], a1, b[0], b[1]);
                hl_mma(acc[1][n + 1], a1, b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int n = n0 + warp * 32 + (lane >> 2) + 8 * r;
        if (n >= n_tokens) continue;
#pragma unroll
        for (int t = 0; t < MN / 8; ++t) {
            const int j = j0 + t * 8 + 2 * (lane & 3);
            if (j >= J) continue;
            float a = acc[r >> 1][t][2 * (r & 1)], b = acc[r >> 1][t][2 * (r & 1) + 1];
            if (gate) {
                const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gate + (size_t)n * gate_ld + (size_t)h * J + j);
                a *= 1.0f / (1.0f + expf(-__bfloat162float(g.x)));
                b *= 1.0f / (1.0f + expf(-__bfloat162float(g.y)));
            }
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)n * out_ld + out_off + (size_t)h * out_head + j) = __floats2bfloat162_rn(a, b);
        }
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
    const bool vectors = I % 8 == 0 && J % 8 == 0 && x_ld % 8 == 0 && x_off % 8 == 0 && x_head % 8 == 0 && out_ld % 2 == 0 &&
                         out_off % 2 == 0 && out_head % 2 == 0 && gate_ld % 2 == 0 && (uintptr_t)x % 16 == 0 &&
                         (uintptr_t)w % 16 == 0 && (uintptr_t)out % 4 == 0 && (uintptr_t)gate % 4 == 0;
    if (is_bf16 && vectors) {
        const int mn = n_tokens <= 32 ? 16 : 64;
        const dim3 tiles(ceil_div(n_tokens, MT), n_head, ceil_div(J, mn));
        MG_REQUIRE(tiles.z <= 65535, "head_linear: too many outputs");
        const cudaError_t em =
            mn == 16 ? mg_launch(head_linear_mma_kernel<16>, tiles, dim3(128), 0, s, true, (const bf16*)x, x_ld, x_off, x_head,
                                 (const bf16*)w, rows_are_inputs, (const bf16*)gate, gate_ld, (bf16*)out, out_ld, out_off, out_head,
                                 n_tokens, I, J)
                     : mg_launch(head_linear_mma_kernel<64>, tiles, dim3(128), 0, s, true, (const bf16*)x, x_ld, x_off, x_head,
                                 (const bf16*)w, rows_are_inputs, (const bf16*)gate, gate_ld, (bf16*)out, out_ld, out_off, out_head,
                                 n_tokens, I, J);
        if (em != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "head_linear (mma): %s", cudaGetErrorString(em));
        return MG_OK;
    }
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
