// Mixers with a matrix memory per head (gated linear attention, mLSTM), prompt portions: the same
// recurrence as the token-by-token scan of matrix_memory.cu, evaluated chunk by chunk so that all SMs
// work and no step waits for the token before it.  A request's tokens of this step are cut into chunks
// of L (the host lists them: request, first row, count); with b_t the sum of the logarithms of the decays
// from the chunk's first token to t (per key channel for gated linear attention, one number per head for
// the mLSTM), three kernels run:
//
//   1. per (chunk, head), all at once:  U = sum_j diag(exp(b_end - b_j)) k_j [v_j, 1]^T   (what the chunk
//      adds to the state), and b itself for the other two kernels;
//   2. per (request, head), chunk after chunk, element-wise:  S_prev(c) is stored where U(c) was, then
//      S <- diag(exp(b_end)) S + U(c); the request's state slot is read at the start (unless the request
//      is new) and written at the end;
//   3. per (chunk, head), all at once:  o_t = (q_t * exp(b_t))^T S_prev + sum_{j <= t} A_tj v_j,
//      A_tj = sum_d q_t[d] k_j[d] exp(b_t[d] - b_j[d]).
//
// Every exponent is <= 0: decays are only ever applied forward in time, so nothing overflows whatever the
// decays are.  For the mLSTM the input gate i_j enters as exp(i_j) on k_j and everything is held relative to
// the running maximum m of the sequential form (m_t = b_t + max(m_prev, max_{j <= t}(i_j - b_j)) inside a chunk;
// a chunk's U is held relative to its own maximum and rescaled in kernel 2), and the normaliser is the
// value column "1": n_t . q_t is that column's output and goes to `aux` with m_t, as in the sequential scan.
// All sums, decays, exponentials and the state are 32-bit; only q, k and v arrive in the compute type.
//
// State-space duality (Mamba-2) runs through the kernels of gated linear attention: its decay exp(-exp(A_h) dt_t)
// is one number per head and token, which is a decay per key channel that happens to be the same in all of
// them.  What differs is read where the rows are loaded (`ssd`): the logarithm of the decay is -exp(A_h) dt_t with
// dt_t = softplus(gates[t, h]), the values enter the memory as dt_t x_t, queries are not scaled, q and k (the C and
// B of the state-space form) are shared by `qk_group` neighbouring heads, and D_h x_t is added to the output.
//
// Retention (`form` 3) is the same with one fixed decay a_h per head: the logarithm of the decay is log(a_h) at every
// token, keys are scaled by head_dim^(-1/2) and queries are not.  The wkv form (`form` 4; RWKV-6 time mixing) has a
// decay exp(-exp(z_t)) per key channel like gated linear attention, but reads BEFORE it updates: o_t = (S_(t-1) +
// diag(u) k_t v_t^T)^T q_t.  So in kernel 3 the query of token t sees the state and the chunk's earlier tokens through
// b_(t-1) instead of b_t (b_(-1) = 0), and its own token through the bonus u alone: A_tt = sum_d q_t[d] u[d] k_t[d].
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(matrix_memory_chunked)

namespace {

constexpr int THREADS = 512;        // kernels 1 and 3: one CTA of 16 warps per SM hides its own latencies
constexpr int SCAN_THREADS = 256;   // kernel 2
constexpr int SCAN_AHEAD = 8;       // chunks whose loads are in flight at once in kernel 2

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

struct ChunkParams {
    const void* proj; int ld; long long q_off, k_off, v_off;
    const float* gates; int gates_ld;
    const int* chunks;            // [n_chunks, 4]: request, first row, tokens, unused
    const int* req_chunks;        // [n_requests, 2]: first chunk, number of chunks
    const int* req_ctx_before; const int* req_state_slot;
    float* state; long long state_stride;
    float* cum;                   // gla: [n_tokens, H, D] b_t;  mlstm: [n_tokens, H, 2] (b_t, i_t)
    float* chunk_state;           // [n_chunks, H, DvE, D]: U, then S_prev
    float* chunk_meta;            // mlstm: [n_chunks, H, 4]: b_end, the chunk's own maximum, m_prev
    float* out; float* aux;
    int n_chunks, n_requests, n_tokens, n_head, d, dv, L, n_slots;
    float constant;
    int ssd, qk_group;            // the state-space form: q and k columns of head h / qk_group
    int form;                     // 0: gated linear attention, 2: state-space, 3: retention, 4: wkv
    const float* head_consts;     // ssd: [2 H]: A_h, then D_h;  retention: [H] decays;  wkv: [H, D] bonus
};

// ---- kernel 1 ----------------------------------------------------------------------------------------
template <typename T, bool MLSTM>
__global__ void __launch_bounds__(THREADS) chunk_local_kernel(const ChunkParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.d, DvE = p.dv + (MLSTM ? 1 : 0), DvP = (DvE + 7) / 8 * 8, L = p.L;
    float* kt = smem;                           // [L][D + 1]
    float* vs = kt + L * (D + 1);               // [L][DvP]
    float* fc = vs + L * DvP;                   // mlstm: [L] b_j, then [L] i_j;  gla: [L][D + 1] b_j
    __shared__ float b_end_s, own_max_s;
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = p.chunks[4 * c + 1], count = p.chunks[4 * c + 2];
    if (!MG_GUARDED(matrix_memory_chunked, MG_GUARD_ROW, row0 + count - 1, p.n_tokens) || count <= 0 || count > L) return;
    const T* proj = reinterpret_cast<const T*>(p.proj);
    if (!MLSTM) {
        // the logarithms of the decays, all at once; then their running sums, a thread per key channel; then the
        // keys as the chunk's end sees them, all at once again
        const float inv_tau = p.ssd ? 0.f : 1.0f / p.constant;
        const float rate = p.ssd ? expf(p.head_consts[h]) : 0.f;
        const float fixed_la = p.form == 3 ? fmaxf(logf(p.head_consts[h]), -1.0e4f) : 0.f;   // (a decay of 0 stays finite)
        for (int idx = tid; idx < L * D; idx += THREADS) {
            const int j = idx / D, d = idx - j * D;
            float la = 0.f;
            if (j < count)
                la = p.ssd ? -rate * softplus(p.gates[(size_t)(row0 + j) * p.gates_ld + h])
                   : p.form == 3 ? fixed_la
                   : p.form == 4 ? -expf(p.gates[(size_t)(row0 + j) * p.gates_ld + (size_t)h * D + d])
                           : log_sigmoid(p.gates[(size_t)(row0 + j) * p.gates_ld + (size_t)h * D + d]) * inv_tau;
            fc[j * (D + 1) + d] = la;
        }
        __syncthreads();
        for (int d = tid; d < D; d += THREADS) {
            float b = 0.f;
            for (int j = 0; j < L; ++j) {
                b += fc[j * (D + 1) + d];
                fc[j * (D + 1) + d] = b;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < L * D; idx += THREADS) {
            const int j = idx / D, d = idx - j * D;
            const float b = fc[j * (D + 1) + d], b_end = fc[(L - 1) * (D + 1) + d];
            float kv = 0.f;
            if (j < count) {
                p.cum[((size_t)(row0 + j) * p.n_head + h) * D + d] = b;
                kv = to_float(proj[(size_t)(row0 + j) * p.ld + p.k_off + (size_t)(h / p.qk_group) * D + d]) * expf(b_end - b);
                if (p.form == 3) kv *= 1.0f / sqrtf((float)D);
            }
            kt[j * (D + 1) + d] = kv;
        }
    } else {
        if (tid < L) {                                          // the two gates of every token, all at once
            float gi = 0.f, lf = 0.f;
            if (tid < count) {
                const float* g = p.gates + (size_t)(row0 + tid) * p.gates_ld;
                gi = p.constant * tanhf(g[h] / p.constant);
                lf = log_sigmoid(p.constant * tanhf(g[p.n_head + h] / p.constant));
            }
            fc[tid] = lf;
            fc[L + tid] = gi;
        }
        __syncthreads();
        if (tid == 0) {
            float b = 0.f, best = -INFINITY;
            for (int j = 0; j < count; ++j) {
                b += fc[j];
                fc[j] = b;
                best = fmaxf(best, fc[L + j] - b);
            }
            b_end_s = b;
            own_max_s = b + best;                               // the largest exponent of the chunk's own tokens at its end
            p.chunk_meta[((size_t)c * p.n_head + h) * 4] = b;
            p.chunk_meta[((size_t)c * p.n_head + h) * 4 + 1] = b + best;
        }
        __syncthreads();
        if (tid < count) {
            p.cum[((size_t)(row0 + tid) * p.n_head + h) * 2] = fc[tid];
            p.cum[((size_t)(row0 + tid) * p.n_head + h) * 2 + 1] = fc[L + tid];
        }
        for (int idx = tid; idx < L * D; idx += THREADS) {
            const int j = idx / D, d = idx - j * D;
            float kv = 0.f;
            if (j < count)
                kv = to_float(proj[(size_t)(row0 + j) * p.ld + p.k_off + (size_t)h * D + d]) *
                     expf(b_end_s - fc[j] + fc[L + j] - own_max_s);
            kt[j * (D + 1) + d] = kv;
        }
    }
    for (int idx = tid; idx < L * DvP; idx += THREADS) {
        const int j = idx / DvP, e = idx - j * DvP;
        float vv = 0.f;
        if (j < count) {
            if (e < p.dv) vv = to_float(proj[(size_t)(row0 + j) * p.ld + p.v_off + (size_t)h * p.dv + e]);
            else if (MLSTM && e == p.dv) vv = 1.f;
            if (!MLSTM && p.ssd) vv *= softplus(p.gates[(size_t)(row0 + j) * p.gates_ld + h]);
        }
        vs[idx] = vv;
    }
    __syncthreads();
    float* U = p.chunk_state + ((size_t)c * p.n_head + h) * DvE * D;
    const int items = (DvP / 8) * D;
    for (int item = tid; item < items; item += THREADS) {
        const int e0 = (item / D) * 8, d = item - (item / D) * D;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < count; ++j) {
            const float kv = kt[j * (D + 1) + d];
            const float4 v0 = *reinterpret_cast<const float4*>(&vs[j * DvP + e0]);
            const float4 v1 = *reinterpret_cast<const float4*>(&vs[j * DvP + e0 + 4]);
            acc[0] = fmaf(kv, v0.x, acc[0]); acc[1] = fmaf(kv, v0.y, acc[1]);
            acc[2] = fmaf(kv, v0.z, acc[2]); acc[3] = fmaf(kv, v0.w, acc[3]);
            acc[4] = fmaf(kv, v1.x, acc[4]); acc[5] = fmaf(kv, v1.y, acc[5]);
            acc[6] = fmaf(kv, v1.z, acc[6]); acc[7] = fmaf(kv, v1.w, acc[7]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (e0 + u < DvE) U[(size_t)(e0 + u) * D + d] = acc[u];
    }
}

// ---- kernel 2 ----------------------------------------------------------------------------------------
template <bool MLSTM>
__global__ void __launch_bounds__(SCAN_THREADS) chunk_scan_kernel(const ChunkParams p) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.z, h = blockIdx.y;
    const int D = p.d, DvE = p.dv + (MLSTM ? 1 : 0);
    const int idx = blockIdx.x * SCAN_THREADS + threadIdx.x;              // element (e, d) of the head's state
    const int first = p.req_chunks[2 * r], n = p.req_chunks[2 * r + 1];
    if (n <= 0) return;
    int slot = p.req_state_slot[r];
    if (!MG_GUARDED(matrix_memory_chunked, MG_GUARD_ROW, slot, p.n_slots) ||
        !MG_GUARDED(matrix_memory_chunked, MG_GUARD_ROW, first + n - 1, p.n_chunks))
        return;
    const bool fresh = p.req_ctx_before[r] == 0;
    const bool mine = idx < DvE * D;
    const int d = mine ? idx % D : 0;
    float* slot_base = p.state + (size_t)slot * p.state_stride;
    float* s_ptr = slot_base + (size_t)h * DvE * D + (mine ? idx : 0);
    float* m_ptr = slot_base + (size_t)p.n_head * DvE * D + h;
    float S = (mine && !fresh) ? *s_ptr : 0.f;
    float m = (MLSTM && !fresh) ? *m_ptr : 0.f;
    for (int c0 = first; c0 < first + n; c0 += SCAN_AHEAD) {
        float U[SCAN_AHEAD];
#pragma unroll
        for (int u = 0; u < SCAN_AHEAD; ++u)                            // several chunks' loads in flight at once
            U[u] = (mine && c0 + u < first + n) ? p.chunk_state[((size_t)(c0 + u) * p.n_head + h) * DvE * D + idx] : 0.f;
#pragma unroll
        for (int u = 0; u < SCAN_AHEAD; ++u) {
            const int c = c0 + u;
            if (c >= first + n) break;
            if (mine) p.chunk_state[((size_t)c * p.n_head + h) * DvE * D + idx] = S;
            if (MLSTM) {
                float* meta = p.chunk_meta + ((size_t)c * p.n_head + h) * 4;
                const float b_end = meta[0], own = meta[1];
                const float m_end = fmaxf(b_end + m, own);
                if (blockIdx.x == 0 && threadIdx.x == 0) meta[2] = m;
                S = expf(b_end + m - m_end) * S + expf(own - m_end) * U[u];
                m = m_end;
            } else {
                const int last = p.chunks[4 * c + 1] + p.chunks[4 * c + 2] - 1;
                S = fmaf(expf(p.cum[((size_t)last * p.n_head + h) * D + d]), S, U[u]);
            }
        }
    }
    if (mine) *s_ptr = S;
    if (MLSTM && blockIdx.x == 0 && threadIdx.x == 0) *m_ptr = m;
}

// ---- kernel 3 ----------------------------------------------------------------------------------------
template <typename T, bool MLSTM>
__global__ void __launch_bounds__(THREADS) chunk_output_kernel(const ChunkParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.d, Dv = p.dv, DvE = Dv + (MLSTM ? 1 : 0), L = p.L;
    const int SP = DvE + 1;                                          // stride of the staged state: odd, conflict-free
    float* qs = smem;                           // [L][D + 1]
    float* ks = qs + L * (D + 1);               // [L][D + 1]
    float* bs = ks + L * (D + 1);               // gla: [L][D + 1];  mlstm: [3 L]: b, i, m
    float* vs = bs + (MLSTM ? 3 * L : L * (D + 1));   // [L][Dv]
    float* As = vs + L * Dv;                    // [L][L + 1]
    float* Ss = As + L * (L + 1);               // [D][SP]: the state before the chunk, transposed
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row0 = p.chunks[4 * c + 1], count = p.chunks[4 * c + 2];
    if (!MG_GUARDED(matrix_memory_chunked, MG_GUARD_ROW, row0 + count - 1, p.n_tokens) || count <= 0 || count > L) return;
    const T* proj = reinterpret_cast<const T*>(p.proj);
    const bool ssd = !MLSTM && p.ssd;
    const bool wkv = !MLSTM && p.form == 4;
    const float q_scale = (ssd || (!MLSTM && p.form >= 3)) ? 1.0f : 1.0f / sqrtf((float)D);
    const float k_scale = (!MLSTM && p.form == 3) ? 1.0f / sqrtf((float)D) : 1.0f;
    const int hq = h / p.qk_group;
    for (int idx = tid; idx < L * D; idx += THREADS) {
        const int j = idx / D, d = idx - j * D;
        float qv = 0.f, kv = 0.f, bv = 0.f;
        if (j < count) {
            const T* row = proj + (size_t)(row0 + j) * p.ld + (size_t)hq * D + d;
            qv = to_float(row[p.q_off]) * q_scale;
            kv = to_float(row[p.k_off]) * k_scale;
            if (!MLSTM) bv = p.cum[((size_t)(row0 + j) * p.n_head + h) * D + d];
        }
        qs[j * (D + 1) + d] = qv;
        ks[j * (D + 1) + d] = kv;
        if (!MLSTM) bs[j * (D + 1) + d] = bv;
    }
    for (int idx = tid; idx < L * Dv; idx += THREADS) {
        const int j = idx / Dv, e = idx - j * Dv;
        float vv = j < count ? to_float(proj[(size_t)(row0 + j) * p.ld + p.v_off + (size_t)h * Dv + e]) : 0.f;
        if (ssd && j < count) vv *= softplus(p.gates[(size_t)(row0 + j) * p.gates_ld + h]);
        vs[idx] = vv;
    }
    const float* S_prev = p.chunk_state + ((size_t)c * p.n_head + h) * DvE * D;
    for (int idx = tid; idx < DvE * D; idx += THREADS) {
        const int e = idx / D, d = idx - e * D;
        Ss[d * SP + e] = S_prev[idx];
    }
    float m_prev = 0.f;
    if (MLSTM) {
        m_prev = p.chunk_meta[((size_t)c * p.n_head + h) * 4 + 2];
        if (tid < L) {
            bs[tid] = tid < count ? p.cum[((size_t)(row0 + tid) * p.n_head + h) * 2] : 0.f;
            bs[L + tid] = tid < count ? p.cum[((size_t)(row0 + tid) * p.n_head + h) * 2 + 1] : 0.f;
        }
        __syncthreads();
        if (tid == 0) {
            float best = -INFINITY;
            for (int j = 0; j < L; ++j) {
                if (j < count) best = fmaxf(best, bs[L + j] - bs[j]);
                bs[2 * L + j] = bs[j] + fmaxf(m_prev, best);        // m_t
            }
        }
    }
    __syncthreads();
    // scores of the chunk's own tokens
    for (int idx = tid; idx < L * (L + 1); idx += THREADS) As[idx] = 0.f;
    __syncthreads();
    // (rows t and L - 1 - t have L + 1 visible keys between them: a pair of rows is one run of L + 1 entries)
    for (int idx = tid; idx < (L / 2) * (L + 1); idx += THREADS) {
        const int pair = idx / (L + 1), k = idx - pair * (L + 1);
        const int t = k <= pair ? pair : L - 1 - pair, j = k <= pair ? k : k - pair - 1;
        if (t >= count) continue;
        float a = 0.f;
        {
            const float* qr = qs + t * (D + 1);
            const float* kr = ks + j * (D + 1);
            if (MLSTM) {
                for (int d = 0; d < D; ++d) a = fmaf(qr[d], kr[d], a);
                a *= __expf(bs[t] - bs[j] + bs[L + j] - bs[2 * L + t]);
            } else if (wkv) {
                if (j == t) {                                        // the token itself: the bonus in place of a decay
                    const float* u = p.head_consts + (size_t)h * D;
                    for (int d = 0; d < D; ++d) a = fmaf(qr[d] * kr[d], u[d], a);
                } else {                                             // the state before token t: decays up to t - 1
                    const float* bt = bs + (t - 1) * (D + 1);
                    const float* bj = bs + j * (D + 1);
                    for (int d = 0; d < D; ++d) a = fmaf(qr[d] * kr[d], __expf(bt[d] - bj[d]), a);
                }
            } else {
                const float* bt = bs + t * (D + 1);
                const float* bj = bs + j * (D + 1);
                for (int d = 0; d < D; ++d) a = fmaf(qr[d] * kr[d], __expf(bt[d] - bj[d]), a);
            }
        }
        As[t * (L + 1) + j] = a;
    }
    __syncthreads();
    // the queries as the state before the chunk sees them
    for (int idx = tid; idx < L * D; idx += THREADS) {
        const int t = idx / D, d = idx - t * D;
        const float f = MLSTM ? __expf(bs[t] + m_prev - bs[2 * L + t])
                      : wkv ? (t > 0 ? __expf(bs[(t - 1) * (D + 1) + d]) : 1.f) : __expf(bs[t * (D + 1) + d]);
        qs[t * (D + 1) + d] *= f;
    }
    __syncthreads();
    // o[t][e]: a warp takes four rows and 128 columns at a time, a lane four of the columns (32 apart)
    const int warp = tid >> 5, lane = tid & 31;
    const int col_groups = (Dv + 127) / 128;
    for (int item = warp; item < (L / 4) * col_groups; item += THREADS / 32) {
        const int t0 = (item / col_groups) * 4, e0 = (item % col_groups) * 128 + lane;
        if (t0 >= count) continue;
        float acc[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
        int e[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) e[x] = min(e0 + 32 * x, Dv - 1);      // (columns beyond the last repeat it; not stored)
        const int j_end = min(t0 + 3, count - 1);
        for (int j = 0; j <= j_end; ++j) {
            float a[4], vv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) a[u] = As[(t0 + u) * (L + 1) + j];
#pragma unroll
            for (int x = 0; x < 4; ++x) vv[x] = vs[j * Dv + e[x]];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[u][x] = fmaf(a[u], vv[x], acc[u][x]);
        }
        for (int d = 0; d < D; ++d) {
            float qv[4], sv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) qv[u] = qs[(t0 + u) * (D + 1) + d];
#pragma unroll
            for (int x = 0; x < 4; ++x) sv[x] = Ss[d * SP + e[x]];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int x = 0; x < 4; ++x) acc[u][x] = fmaf(qv[u], sv[x], acc[u][x]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int x = 0; x < 4; ++x)
                if (t0 + u < count && e0 + 32 * x < Dv) {
                    float o = acc[u][x];
                    if (ssd)                                          // D_h x_t, with x_t as it arrived
                        o = fmaf(p.head_consts[p.n_head + h],
                                 to_float(proj[(size_t)(row0 + t0 + u) * p.ld + p.v_off + (size_t)h * Dv + e0 + 32 * x]), o);
                    p.out[((size_t)(row0 + t0 + u) * p.n_head + h) * Dv + e0 + 32 * x] = o;
                }
    }
    if (MLSTM && tid < count) {                                       // the normaliser's column, a row a thread
        const int t = tid;
        float nq = 0.f;
        for (int j = 0; j <= t; ++j) nq += As[t * (L + 1) + j];
        for (int d = 0; d < D; ++d) nq = fmaf(qs[t * (D + 1) + d], Ss[d * SP + Dv], nq);
        p.aux[((size_t)(row0 + t) * p.n_head + h) * 2] = nq;
        p.aux[((size_t)(row0 + t) * p.n_head + h) * 2 + 1] = bs[2 * L + t];
    }
}

size_t local_smem(int L, int D, int DvE, bool mlstm) {
    return sizeof(float) * ((size_t)L * (D + 1) + (size_t)L * ((DvE + 7) / 8 * 8) + (mlstm ? 2 * L : (size_t)L * (D + 1)));
}
size_t output_smem(int L, int D, int Dv, bool mlstm) {
    const int DvE = Dv + (mlstm ? 1 : 0);
    return sizeof(float) * ((size_t)2 * L * (D + 1) + (mlstm ? 3 * L : (size_t)L * (D + 1)) + (size_t)L * Dv +
                            (size_t)L * (L + 1) + (size_t)D * (DvE + 1));
}
constexpr size_t SMEM_LIMIT = 200 * 1024;

template <typename T, bool MLSTM>
int run_chunked(const ChunkParams& p, cudaStream_t s) {
    const int DvE = p.dv + (MLSTM ? 1 : 0);
    const size_t s1 = local_smem(p.L, p.d, DvE, MLSTM), s3 = output_smem(p.L, p.d, p.dv, MLSTM);
    cudaError_t e = cudaFuncSetAttribute(chunk_local_kernel<T, MLSTM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(chunk_output_kernel<T, MLSTM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "matrix memory (chunks): %s", cudaGetErrorString(e));
    e = mg_launch(chunk_local_kernel<T, MLSTM>, dim3(p.n_chunks, p.n_head), dim3(THREADS), s1, s, true, p);
    if (e == cudaSuccess)
        e = mg_launch(chunk_scan_kernel<MLSTM>, dim3(ceil_div(DvE * p.d, SCAN_THREADS), p.n_head, p.n_requests), dim3(SCAN_THREADS), 0, s, true, p);
    if (e == cudaSuccess)
        e = mg_launch(chunk_output_kernel<T, MLSTM>, dim3(p.n_chunks, p.n_head), dim3(THREADS), s3, s, true, p);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "matrix memory (chunks): %s", cudaGetErrorString(e));
    return MG_OK;
}

}  // namespace

// The longest chunk (64 or 32 tokens) whose tiles fit the shared memory of an SM for heads of these sizes;
// 0 if none does (then the sequential scan serves).
MG_API int mg_matrix_memory_chunk_tokens(int head_dim, int v_dim, int mlstm) {
    for (int L = 64; L >= 32; L /= 2)
        if (output_smem(L, head_dim, v_dim, mlstm != 0) <= SMEM_LIMIT && local_smem(L, head_dim, v_dim + 1, mlstm != 0) <= SMEM_LIMIT)
            return L;
    return 0;
}

// As mg_matrix_memory_scan (same rows, gates, state slots, out and aux), for steps with prompt portions.
// chunks: [n_chunks, 4] (request, first row, tokens <= chunk_tokens, unused) in row order; req_chunks:
// [n_requests, 2] (first chunk, chunks); cum: [n_tokens, n_head, mlstm ? 2 : head_dim] floats; chunk_state:
// [n_chunks, n_head, v_dim + mlstm, head_dim] floats; chunk_meta: [n_chunks, n_head, 4] floats (mlstm; else null).
// qk_group > 0 with head_consts ([A_0 .. A_(H-1), D_0 .. D_(H-1)], 32-bit): the state-space form (not with mlstm);
// gates then hold one step size per head before its softplus, and `state` points at the memories of slot 0.
// form 3 (retention: head_consts = [H] decays, no gates) and 4 (wkv: head_consts = [H, D] bonus, gates = the decays'
// pre-activations [tokens, H * D]); 0: as said above.  Offsets beyond a row name planes, as in mg_matrix_memory_scan.
MG_API int mg_matrix_memory_chunked(const void* proj, int ld, long long q_off, long long k_off, long long v_off, const float* gates,
                                    int gates_ld, const int* chunks, const int* req_chunks, const int* req_ctx_before,
                                    const int* req_state_slot, float* state, long long state_stride, float* cum,
                                    float* chunk_state, float* chunk_meta, float* out, float* aux, int n_chunks,
                                    int chunk_tokens, int n_requests, int n_tokens, int n_head, int head_dim, int v_dim,
                                    float constant, int mlstm, int n_slots, int is_bf16, int qk_group,
                                    const float* head_consts, int form, void* stream) {
    if (n_requests == 0 || n_tokens == 0 || n_chunks == 0) return MG_OK;
    MG_REQUIRE(n_requests > 0 && n_tokens > 0 && n_chunks > 0 && n_head > 0 && head_dim > 0 && v_dim > 0 && n_slots > 0,
               "matrix memory (chunks): bad sizes");
    MG_REQUIRE(n_head <= 65535 && n_requests <= 65535, "matrix memory (chunks): too many heads or requests");
    MG_REQUIRE(form == 0 || ((form == 3 || form == 4) && !mlstm && head_consts != nullptr), "matrix memory (chunks): form %d", form);
    const bool ssd = head_consts != nullptr && form == 0;
    MG_REQUIRE(ssd || form != 0 || constant > 0.f, "matrix memory (chunks): tau and the gates' cap must be positive");
    MG_REQUIRE(!ssd || (!mlstm && qk_group > 0 && n_head % qk_group == 0), "matrix memory (chunks): %d heads do not form groups of %d", n_head, qk_group);
    if (!ssd) qk_group = 1;
    const int qk_heads = n_head / qk_group;
    const int cols = v_dim + (mlstm ? 1 : 0);
    MG_REQUIRE(state_stride >= (long long)n_head * cols * head_dim + (mlstm ? n_head : 0), "matrix memory (chunks): the state slots are too small");
    MG_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off % ld + qk_heads * head_dim <= ld && k_off % ld + qk_heads * head_dim <= ld &&
                   v_off % ld + n_head * v_dim <= ld, "matrix memory (chunks): heads outside the rows");
    MG_REQUIRE(form == 3 || (gates != nullptr && gates_ld >= (mlstm ? 2 * n_head : ssd ? n_head : n_head * head_dim)),
               "matrix memory (chunks): the gates' rows are too short");
    MG_REQUIRE(cum && chunk_state && (!mlstm || (chunk_meta && aux)), "matrix memory (chunks): scratch is missing");
    MG_REQUIRE((chunk_tokens == 32 || chunk_tokens == 64) && chunk_tokens <= mg_matrix_memory_chunk_tokens(head_dim, v_dim, mlstm),
               "matrix memory (chunks): chunks of %d tokens do not fit heads of %d and %d", chunk_tokens, head_dim, v_dim);
    ChunkParams p;
    p.proj = proj; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.gates = gates; p.gates_ld = gates_ld;
    p.chunks = chunks; p.req_chunks = req_chunks; p.req_ctx_before = req_ctx_before; p.req_state_slot = req_state_slot;
    p.state = state; p.state_stride = state_stride; p.cum = cum; p.chunk_state = chunk_state; p.chunk_meta = chunk_meta;
    p.out = out; p.aux = aux; p.n_chunks = n_chunks; p.n_requests = n_requests; p.n_tokens = n_tokens; p.n_head = n_head;
    p.d = head_dim; p.dv = v_dim; p.L = chunk_tokens; p.n_slots = n_slots; p.constant = constant;
    p.ssd = ssd ? 1 : 0; p.qk_group = qk_group; p.head_consts = head_consts; p.form = ssd ? 2 : form;
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16) return mlstm ? run_chunked<bf16, true>(p, s) : run_chunked<bf16, false>(p, s);
    return mlstm ? run_chunked<float, true>(p, s) : run_chunked<float, false>(p, s);
}
