// Mixers with a matrix memory per head that is carried from token to token (gated linear attention,
// mLSTM): the scan over a step's tokens, and the norm and gate of the heads that follows it.
//
// scan, per request r and head h, for the request's tokens t in order:
//   gated linear attention:  S <- diag(a_t) S + k_t v_t^T,  a_t = sigmoid(z_t)^(1/tau)  (per key channel)
//   mLSTM:                   m' = max(f_t + m, i_t),  S <- exp(f_t + m - m') S + exp(i_t - m') k_t [v_t, 1]^T,
//                            i_t = cap tanh(x_i / cap),  f_t = logsigmoid(cap tanh(x_f / cap))
//   state-space duality (Mamba-2):  S <- exp(-exp(A_h) dt_t) S + dt_t B_t x_t^T,  dt_t = softplus(raw dt_t),
//                            o_t = S^T C_t + D_h x_t; B and C (in the places of k and q, unscaled) are shared by the
//                            heads of a group of neighbouring heads, A_h and D_h are one number per head
//   retention:               S <- a_h S + (k_t / sqrt(head_dim)) v_t^T with one fixed decay a_h per head (q unscaled)
//   wkv (RWKV-6 time mixing): o_t = (S + diag(u_h) k_t v_t^T)^T q_t is read BEFORE the update (the bonus u weighs the
//                            current token only), then S <- diag(w_t) S + k_t v_t^T, w_t = exp(-exp(z_t)) per key
//                            channel; q and k unscaled
//   o_t = S^T q_t,  q_t scaled by head_dim^(-1/2) (first two forms)
// S is [value column][key channel] in 32-bit in the request's state slot; it starts at zero when the
// request has nothing in the cache.  For the mLSTM the normaliser n is one more value column (the
// value 1), whose output n_t . q_t goes to `aux` with m_t; the division happens in the second kernel.
//
// One CTA owns 32 value columns of one (request, head); four threads share a column, each holding a
// quarter of the key channels in registers.  A token costs head_dim / 4 multiply-adds per thread for
// the update and as many for the read, then two shuffles; q, k and the decays of 16 tokens at a time
// are staged in shared memory (8 at a time for the largest heads) (decays, gates and exponentials evaluated there, once, in 32-bit).  The
// order of every sum is fixed, so a token's result does not depend on how its request was cut into
// steps or on what else is in the batch.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(matrix_memory)

namespace {

constexpr int COLS = 32;                 // value columns per CTA
constexpr int DPARTS = 4;                // threads per column
constexpr int THREADS = COLS * DPARTS;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// DPT: key channels per thread (head_dim <= 4 * DPT; channels beyond head_dim are zeros)
constexpr int MODE_GLA = 0, MODE_MLSTM = 1, MODE_SSD = 2, MODE_RETENTION = 3, MODE_WKV = 4;

__device__ __forceinline__ float softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <typename T, int DPT, int MODE>
__global__ void __launch_bounds__(THREADS)
matrix_memory_scan_kernel(const T* __restrict__ proj, int ld, long long q_off, long long k_off, long long v_off,
                          const float* __restrict__ gates, int gates_ld, const int* __restrict__ req_q_start,
                          const int* __restrict__ req_q_len, const int* __restrict__ req_ctx_before,
                          const int* __restrict__ req_state_slot, float* __restrict__ state, long long state_stride,
                          float* __restrict__ out, float* __restrict__ aux, int n_head, int head_dim, int v_dim,
                          float constant, int n_slots, int n_tokens, int qk_group, const float* __restrict__ head_consts) {
    constexpr bool MLSTM = MODE == MODE_MLSTM, SSD = MODE == MODE_SSD, WKV = MODE == MODE_WKV, RET = MODE == MODE_RETENTION;
    constexpr bool GLA = MODE == MODE_GLA || WKV;              // one decay per key channel and token
    constexpr int TCHUNK = DPT >= 64 ? 8 : 16;                 // tokens staged at a time (48 KB of shared memory at most)
    constexpr int ROW = DPT + 4;                               // a thread's channels, padded: float4 reads without bank conflicts
    __shared__ __align__(16) float q_s[TCHUNK][DPARTS * ROW];
    __shared__ __align__(16) float k_s[TCHUNK][DPARTS * ROW];
    __shared__ __align__(16) float a_s[GLA ? TCHUNK : 1][GLA ? DPARTS * ROW : 4];
    __shared__ float v_s[TCHUNK][COLS];
    __shared__ __align__(16) float u_s[WKV ? DPARTS * ROW : 4];     // wkv: the bonus of the head's key channels
    __shared__ float gi_s[TCHUNK], gf_s[TCHUNK];
    pdl_trigger();
    pdl_wait();                                                // the projections come from the kernels in front
    const int r = blockIdx.z, h = blockIdx.y, slice = blockIdx.x;
    const int q_len = req_q_len[r];
    if (q_len <= 0) return;                                    // a padding row of a fixed-size batch
    const int start = req_q_start[r];
    int slot = req_state_slot[r];
    if (!MG_GUARDED(matrix_memory, MG_GUARD_ROW, slot, n_slots) ||
        !MG_GUARDED(matrix_memory, MG_GUARD_ROW, start + q_len - 1, n_tokens))
        return;
    const bool fresh = req_ctx_before[r] == 0;
    const int tid = threadIdx.x, col_local = tid / DPARTS, dpart = tid % DPARTS;
    const int cols_total = v_dim + (MLSTM ? 1 : 0);
    const int col = slice * COLS + col_local;
    const bool col_ok = col < cols_total;
    float* slot_base = state + (size_t)slot * state_stride;
    float* s_base = slot_base + ((size_t)h * cols_total + (col_ok ? col : 0)) * head_dim;
    float* m_ptr = slot_base + (size_t)n_head * cols_total * head_dim + h;

    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = dpart * DPT + i;
        S[i] = (!fresh && col_ok && d < head_dim) ? s_base[d] : 0.f;
    }
    float m = (MLSTM && !fresh) ? *m_ptr : 0.f;
    const float q_scale = (SSD || RET || WKV) ? 1.0f : 1.0f / sqrtf((float)head_dim);
    const float k_scale = RET ? 1.0f / sqrtf((float)head_dim) : 1.0f;
    const float inv_tau = (GLA && !WKV) ? 1.0f / constant : 0.f;
    const float fixed_keep = RET ? head_consts[h] : 1.f;
    if (WKV) {
        for (int d = tid; d < DPARTS * DPT; d += THREADS)
            u_s[(d / DPT) * ROW + (d % DPT)] = d < head_dim ? head_consts[(size_t)h * head_dim + d] : 0.f;
    }
    const int hq = h / qk_group;                               // the head whose q and k columns this head reads
    const float rate = SSD ? expf(head_consts[h]) : 0.f, skip = SSD ? head_consts[n_head + h] : 0.f;

    for (int t0 = 0; t0 < q_len; t0 += TCHUNK) {
        const int nt = min(TCHUNK, q_len - t0);
        __syncthreads();                                       // the chunk before is used up
        for (int idx = tid; idx < nt * DPARTS * DPT; idx += THREADS) {
            const int tt = idx / (DPARTS * DPT), d = idx - tt * (DPARTS * DPT);
            const size_t token = (size_t)(start + t0 + tt);
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (d < head_dim) {
                const T* row = proj + token * ld + (size_t)hq * head_dim + d;
                qv = to_float(row[q_off]) * q_scale;
                kv = to_float(row[k_off]) * k_scale;
                if (WKV) av = expf(-expf(gates[token * gates_ld + (size_t)h * head_dim + d]));
                else if (GLA) av = expf(log_sigmoid(gates[token * gates_ld + (size_t)h * head_dim + d]) * inv_tau);
            }
            const int at = (d / DPT) * ROW + (d % DPT);
            q_s[tt][at] = qv;
            k_s[tt][at] = kv;
            if (GLA) a_s[tt][at] = av;
        }
        for (int idx = tid; idx < nt * COLS; idx += THREADS) {
            const int tt = idx / COLS, c = idx - tt * COLS, cg = slice * COLS + c;
            const size_t token = (size_t)(start + t0 + tt);
            float vv = 0.f;
            if (cg < v_dim) vv = to_float(proj[token * ld + v_off + (size_t)h * v_dim + cg]);
            else if (MLSTM && cg == v_dim) vv = 1.f;           // the normaliser's column
            v_s[tt][c] = vv;
        }
        if (MLSTM && tid < nt) {
            const float* g = gates + (size_t)(start + t0 + tid) * gates_ld;
            gi_s[tid] = constant * tanhf(g[h] / constant);
            gf_s[tid] = log_sigmoid(constant * tanhf(g[n_head + h] / constant));
        }
        if (SSD && tid < nt) {
            const float dt = softplus(gates[(size_t)(start + t0 + tid) * gates_ld + h]);
            gi_s[tid] = dt;                                    // the step size
            gf_s[tid] = expf(-rate * dt);                      // what the state keeps over the step
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float keep = fixed_keep, vv = v_s[tt][col_local];
            if (MLSTM) {
                const float gi = gi_s[tt], gf = gf_s[tt];
                const float m_new = fmaxf(gf + m, gi);
                keep = expf(gf + m - m_new);
                vv *= expf(gi - m_new);
                m = m_new;
            }
            const float x_raw = vv;
            if (SSD) {
                keep = gf_s[tt];
                vv *= gi_s[tt];
            }
            const float4* q4 = reinterpret_cast<const float4*>(&q_s[tt][dpart * ROW]);
            const float4* k4 = reinterpret_cast<const float4*>(&k_s[tt][dpart * ROW]);
            const float4* a4 = reinterpret_cast<const float4*>(&a_s[GLA ? tt : 0][GLA ? dpart * ROW : 0]);
            float acc = 0.f;
            if (WKV) {
                // the read comes first and sees the state before this token, plus the token's own k v^T weighed by u
                const float4* u4 = reinterpret_cast<const float4*>(&u_s[dpart * ROW]);
                float bonus = 0.f;
#pragma unroll
                for (int i = 0; i < DPT; i += 4) {
                    const float4 qv = q4[i / 4], kv = k4[i / 4], av = a4[i / 4], uv = u4[i / 4];
                    acc = fmaf(S[i], qv.x, acc);
                    acc = fmaf(S[i + 1], qv.y, acc);
                    acc = fmaf(S[i + 2], qv.z, acc);
                    acc = fmaf(S[i + 3], qv.w, acc);
                    bonus = fmaf(qv.x * uv.x, kv.x, bonus);
                    bonus = fmaf(qv.y * uv.y, kv.y, bonus);
                    bonus = fmaf(qv.z * uv.z, kv.z, bonus);
                    bonus = fmaf(qv.w * uv.w, kv.w, bonus);
                    S[i] = fmaf(av.x, S[i], kv.x * vv);
                    S[i + 1] = fmaf(av.y, S[i + 1], kv.y * vv);
                    S[i + 2] = fmaf(av.z, S[i + 2], kv.z * vv);
                    S[i + 3] = fmaf(av.w, S[i + 3], kv.w * vv);
                }
                acc = fmaf(bonus, vv, acc);
            } else
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 qv = q4[i / 4], kv = k4[i / 4];
                float4 av = make_float4(keep, keep, keep, keep);
                if (GLA) av = a4[i / 4];
                S[i] = fmaf(av.x, S[i], kv.x * vv);
                S[i + 1] = fmaf(av.y, S[i + 1], kv.y * vv);
                S[i + 2] = fmaf(av.z, S[i + 2], kv.z * vv);
                S[i + 3] = fmaf(av.w, S[i + 3], kv.w * vv);
                acc = fmaf(S[i], qv.x, acc);
                acc = fmaf(S[i + 1], qv.y, acc);
                acc = fmaf(S[i + 2], qv.z, acc);
                acc = fmaf(S[i + 3], qv.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (dpart == 0 && col_ok) {
                const size_t token = (size_t)(start + t0 + tt);
                if (col < v_dim) out[(token * n_head + h) * v_dim + col] = SSD ? fmaf(skip, x_raw, acc) : acc;
                else {
                    aux[(token * n_head + h) * 2] = acc;       // n_t . q_t
                    aux[(token * n_head + h) * 2 + 1] = m;     // m_t
                }
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = dpart * DPT + i;
            if (d < head_dim) s_base[d] = S[i];
        }
    }
    if (MLSTM && slice == 0 && tid == 0) *m_ptr = m;
}

constexpr int NORM_WARPS = 4;

// out[t, h, :] = (o / den) / rms(o / den) * gain * act(gate), one warp per (token, head); den = 1 without aux.
template <typename T>
__global__ void __launch_bounds__(32 * NORM_WARPS)
head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ aux, const T* __restrict__ gate, int gate_ld,
                      const float* __restrict__ gain, const int* __restrict__ positions, T* __restrict__ out, int n_head,
                      int v_dim, float eps, int per_head_gain, int gate_sigmoid) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x, h = blockIdx.y * NORM_WARPS + warp;
    if (h >= n_head) return;
    T* orow = out + ((size_t)token * n_head + h) * v_dim;
    if (positions != nullptr && positions[token] < 0) {        // padding: nothing was computed for it
        for (int d = lane; d < v_dim; d += 32) orow[d] = from_float<T>(0.f);
        return;
    }
    const float* src = o + ((size_t)token * n_head + h) * v_dim;
    float inv_den = 1.f;
    if (aux != nullptr) {
        const float nq = aux[((size_t)token * n_head + h) * 2], m = aux[((size_t)token * n_head + h) * 2 + 1];
        inv_den = 1.0f / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
    float sq = 0.f;
    for (int d = lane; d < v_dim; d += 32) {
        const float x = src[d] * inv_den;
        sq = fmaf(x, x, sq);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)v_dim + eps);
    const float* gn = gain ? gain + (per_head_gain ? (size_t)h * v_dim : 0) : nullptr;
    const T* grow = gate + (size_t)token * gate_ld + (size_t)h * v_dim;
    for (int d = lane; d < v_dim; d += 32) {
        const float g = to_float(grow[d]);
        const float sg = 1.0f / (1.0f + expf(-g));
        orow[d] = from_float<T>(src[d] * inv_den * rstd * (gn ? gn[d] : 1.f) * (gate_sigmoid ? sg : g * sg));
    }
}

template <typename T, int MODE>
cudaError_t launch_scan(int dpt, dim3 grid, cudaStream_t s, const T* proj, int ld, long long q_off, long long k_off, long long v_off,
                        const float* gates, int gates_ld, const int* q_start, const int* q_len, const int* ctx_before,
                        const int* slots, float* state, long long stride, float* out, float* aux, int n_head,
                        int head_dim, int v_dim, float constant, int n_slots, int n_tokens, int qk_group,
                        const float* head_consts) {
#define MG_SCAN(D)                                                                                                  \
    return mg_launch(matrix_memory_scan_kernel<T, D, MODE>, grid, dim3(THREADS), 0, s, true, proj, ld, q_off, k_off,  \
                     v_off, gates, gates_ld, q_start, q_len, ctx_before, slots, state, stride, out, aux, n_head,      \
                     head_dim, v_dim, constant, n_slots, n_tokens, qk_group, head_consts)
    switch (dpt) {
        case 4: MG_SCAN(4);
        case 8: MG_SCAN(8);
        case 16: MG_SCAN(16);
        case 32: MG_SCAN(32);
        default: MG_SCAN(64);
    }
#undef MG_SCAN
}

}  // namespace

// proj: [n_tokens, ld] rows (bfloat16 if is_bf16 else 32-bit) holding q and k (n_head / qk_group x head_dim each; head
// h reads those of head h / qk_group) and v (n_head x v_dim) at the three column offsets; gates: 32-bit rows of
// gates_ld numbers: mode 0 (gated linear attention; constant = tau) the decays' pre-activations z [n_head x head_dim],
// mode 1 (mLSTM; constant = the cap) the input and forget gates' pre-activations [2 x n_head], mode 2 (state-space
// duality) the step sizes before their softplus [n_head], with head_consts = [A_0 .. A_(H-1), D_0 .. D_(H-1)] 32-bit on
// the device; mode 3 (retention) no gates, head_consts = the decay of every head [n_head]; mode 4 (wkv) the decays'
// pre-activations z [n_head x head_dim] (w = exp(-exp(z))), head_consts = the bonus [n_head x head_dim].  An offset
// of p * n_tokens * ld + c names column c of plane p of a [planes, n_tokens, ld] tensor.  req_*: [n_requests] first row, tokens, tokens already in the cache, state slot.  state: [n_slots,
// state_stride] 32-bit.  out: [n_tokens, n_head * v_dim] 32-bit; aux: [n_tokens, n_head, 2] 32-bit (mLSTM only).
MG_API int mg_matrix_memory_scan(const void* proj, int ld, long long q_off, long long k_off, long long v_off, const float* gates,
                                 int gates_ld, const int* req_q_start, const int* req_q_len, const int* req_ctx_before,
                                 const int* req_state_slot, float* state, long long state_stride, float* out, float* aux,
                                 int n_requests, int n_tokens, int n_head, int head_dim, int v_dim, float constant,
                                 int mode, int n_slots, int is_bf16, int qk_group, const float* head_consts, void* stream) {
    if (n_requests == 0 || n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_requests > 0 && n_tokens > 0 && n_head > 0 && head_dim > 0 && v_dim > 0 && n_slots > 0,
               "matrix memory: bad sizes");
    MG_REQUIRE(mode >= 0 && mode <= 4, "matrix memory: mode %d", mode);
    MG_REQUIRE(head_dim <= 256, "matrix memory: heads of up to 256 key channels (got %d)", head_dim);
    MG_REQUIRE(n_head <= 65535 && n_requests <= 65535, "matrix memory: too many heads or requests");
    MG_REQUIRE(mode >= MODE_SSD || constant > 0.f, "matrix memory: tau and the gates' cap must be positive");
    MG_REQUIRE(qk_group > 0 && n_head % qk_group == 0, "matrix memory: %d heads do not form groups of %d", n_head, qk_group);
    MG_REQUIRE(mode < MODE_SSD || head_consts != nullptr, "matrix memory: this form wants its per-head constants");
    MG_REQUIRE(mode == MODE_RETENTION || gates != nullptr, "matrix memory: this form wants its gates");
    const bool mlstm = mode == MODE_MLSTM;
    const int cols = v_dim + (mlstm ? 1 : 0), qk_heads = n_head / qk_group;
    MG_REQUIRE(state_stride >= (long long)n_head * cols * head_dim + (mlstm ? n_head : 0), "matrix memory: the state slots are too small");
    // (an offset beyond a row names a plane of a [planes, n_tokens, ld] tensor: q, k and v from projections of their own)
    MG_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off % ld + qk_heads * head_dim <= ld && k_off % ld + qk_heads * head_dim <= ld &&
                   v_off % ld + n_head * v_dim <= ld, "matrix memory: heads outside the rows");
    MG_REQUIRE(mode == MODE_RETENTION || gates_ld >= (mlstm ? 2 * n_head : mode == MODE_SSD ? n_head : n_head * head_dim),
               "matrix memory: the gates' rows are too short");
    MG_REQUIRE(!mlstm || aux != nullptr, "matrix memory: the mLSTM wants room for its normaliser");
    const int dpt = head_dim <= 16 ? 4 : head_dim <= 32 ? 8 : head_dim <= 64 ? 16 : head_dim <= 128 ? 32 : 64;
    const dim3 grid(ceil_div(cols, COLS), n_head, n_requests);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
#define MG_SCAN_ARGS(T) dpt, grid, s, (const T*)proj, ld, q_off, k_off, v_off, gates, gates_ld, req_q_start, req_q_len, req_ctx_before, \
                        req_state_slot, state, state_stride, out, aux, n_head, head_dim, v_dim, constant, n_slots, n_tokens, qk_group, head_consts
    if (is_bf16)
        e = mode == MODE_MLSTM ? launch_scan<bf16, MODE_MLSTM>(MG_SCAN_ARGS(bf16))
          : mode == MODE_SSD   ? launch_scan<bf16, MODE_SSD>(MG_SCAN_ARGS(bf16))
          : mode == MODE_RETENTION ? launch_scan<bf16, MODE_RETENTION>(MG_SCAN_ARGS(bf16))
          : mode == MODE_WKV   ? launch_scan<bf16, MODE_WKV>(MG_SCAN_ARGS(bf16))
                               : launch_scan<bf16, MODE_GLA>(MG_SCAN_ARGS(bf16));
    else
        e = mode == MODE_MLSTM ? launch_scan<float, MODE_MLSTM>(MG_SCAN_ARGS(float))
          : mode == MODE_SSD   ? launch_scan<float, MODE_SSD>(MG_SCAN_ARGS(float))
          : mode == MODE_RETENTION ? launch_scan<float, MODE_RETENTION>(MG_SCAN_ARGS(float))
          : mode == MODE_WKV   ? launch_scan<float, MODE_WKV>(MG_SCAN_ARGS(float))
                               : launch_scan<float, MODE_GLA>(MG_SCAN_ARGS(float));
#undef MG_SCAN_ARGS
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "matrix memory scan: %s", cudaGetErrorString(e));
    return MG_OK;
}

// o: [n_tokens, n_head * v_dim] 32-bit; aux: [n_tokens, n_head, 2] or null; gate: rows of gate_ld elements whose
// first n_head * v_dim are the gates' pre-activations; gain: [v_dim], or [n_head * v_dim] if per_head_gain, or null (none);
// positions: [n_tokens] or null; out: [n_tokens, n_head * v_dim] in the gate's type.  gate_sigmoid 1: sigmoid, 0: silu.
MG_API int mg_head_norm_gate(const float* o, const float* aux, const void* gate, int gate_ld, const float* gain,
                             const int* positions, void* out, int n_tokens, int n_head, int v_dim, float eps,
                             int per_head_gain, int gate_sigmoid, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && v_dim > 0 && gate_ld >= n_head * v_dim, "head norm: bad sizes");
    const dim3 grid(n_tokens, ceil_div(n_head, NORM_WARPS)), block(32 * NORM_WARPS);
    MG_REQUIRE(grid.y <= 65535, "head norm: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t e =
        is_bf16 ? mg_launch(head_norm_gate_kernel<bf16>, grid, block, 0, s, true, o, aux, (const bf16*)gate, gate_ld, gain,
                            positions, (bf16*)out, n_head, v_dim, eps, per_head_gain, gate_sigmoid)
                : mg_launch(head_norm_gate_kernel<float>, grid, block, 0, s, true, o, aux, (const float*)gate, gate_ld, gain,
                            positions, (float*)out, n_head, v_dim, eps, per_head_gain, gate_sigmoid);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "head norm: %s", cudaGetErrorString(e));
    return MG_OK;
}
