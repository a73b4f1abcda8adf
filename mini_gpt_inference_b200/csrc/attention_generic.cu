// Causal attention of a ragged batch over the paged cache; the general kernel.
//
// One warp per (token, head).  The token's query attends to the keys of its own request at
// positions lo..p, p being the token's own position and lo = max(0, p - window + 1) (0
// without a window), all read from the request's pages: the keys of this step were written
// there before the launch.  Scores, the running maximum, the running sum and the output
// accumulate in 32-bit; keys are visited in blocks of 32 starting at lo, so the result of a
// (token, head) pair is the same in whichever step and batch it is computed.
//
// Two further masks and biases, both parameters: `block` > 0 lets a query see only the keys of its own
// block of that many positions (lo is raised to the block's first position; blocks are counted from
// position 0 of the sequence); `slopes` (one number per head) takes slope_h * (p - j) off the score
// of key j.
//
// Any key size up to 1,024 and value size up to 512 and any number of heads and kv heads (n_head a
// multiple of n_kv_head) are accepted.  Entries of the block table are read only for positions lo..p, so
// stale or missing pages elsewhere never matter.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(attention_generic)

namespace {

constexpr int WARPS = 4;
constexpr int MAX_KEY_DIM = 1024;   // a warp's query in shared memory
constexpr int MAX_VALUE_DIM = 512;  // value features per lane: 8 (values of up to 256) or 16

template <typename T, int MAX_DPL>
__global__ void __launch_bounds__(32 * WARPS)
paged_attention_generic_kernel(const T* __restrict__ qkv, int q_stride, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               const int* __restrict__ token_request, const int* __restrict__ positions,
                               T* __restrict__ out, int n_tokens, int n_head, int n_kv_head, int head_dim, int v_dim,
                               const T* __restrict__ gate, int gate_stride,
                               int page_tokens, int max_pages, int window, float scale, int num_pages,
                               int n_requests, const float* __restrict__ slopes, int block, float softcap,
                               const float* __restrict__ sinks, int v_stride) {
    extern __shared__ float q_smem[];                     // [WARPS][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    const int head = blockIdx.y * WARPS + warp;
    if (head >= n_head) return;                            // whole warp leaves together
    const int kv_head = head / (n_head / n_kv_head);
    int p = positions[token];
    if (p < 0) {                                           // padding row of a fixed-size batch
        T* pad = out + (size_t)token * n_head * v_dim + (size_t)head * v_dim;
        for (int d = lane; d < v_dim; d += 32) pad[d] = from_float<T>(0.f);
        return;
    }
    // (guarded builds: a position beyond the block table, a request beyond its rows or a page beyond
    // the pool is recorded, and position 0, request 0 or page 0 is read in its place)
    if (!MG_GUARDED(attention_generic, MG_GUARD_POSITION, p, (long long)max_pages * page_tokens)) p = 0;
    int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    if (block > 0) lo = max(lo, p / block * block);
    const float slope = slopes ? slopes[head] : 0.f;
    int request = token_request[token];
    if (!MG_GUARDED(attention_generic, MG_GUARD_REQUEST, request, n_requests)) request = 0;
    const int* table = block_table + (size_t)request * max_pages;

    float* q = q_smem + warp * head_dim;
    const T* qrow = qkv + (size_t)token * q_stride + (size_t)head * head_dim;
    for (int d = lane; d < head_dim; d += 32) q[d] = to_float(qrow[d]) * scale;
    __syncwarp();

    float acc[MAX_DPL];
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[i] = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= p;
        int row = 0;                                       // row of key j in the page storage
        float s = -INFINITY;
        if (valid) {
            int page = table[j / page_tokens];
            if (!MG_GUARDED(attention_generic, MG_GUARD_PAGE, page, num_pages)) page = 0;
            row = (page * n_kv_head + kv_head) * page_tokens + (j % page_tokens);
            const T* kr = k_pages + (size_t)row * head_dim;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(q[d], to_float(kr[d]), dot);
            if (softcap > 0.f) dot = softcap * tanhf(dot / softcap);
            s = slopes ? dot - slope * (float)(p - j) : dot;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float prob = valid ? expf(s - new_max) : 0.f;
        const float corr = expf(run_max - new_max);       // 0 in the first block (run_max = -inf)
        run_sum = run_sum * corr + warp_sum(prob);
        run_max = new_max;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) acc[i] *= corr;
        const int count = min(32, p - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, prob, jj);
            const int rj = __shfl_sync(0xffffffffu, row, jj);
            const T* vr = v_pages + (size_t)rj * v_stride;
#pragma unroll
            for (int i = 0; i < MAX_DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < v_dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
            }
        }
    }
    if (sinks) {
        // a sink: one more term exp(sink_h) in the denominator, with no key and no value
        const float sink = sinks[head];
        const float new_max = fmaxf(run_max, sink);
        const float corr = expf(run_max - new_max);
        run_sum = run_sum * corr + expf(sink - new_max);
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) acc[i] *= corr;
    }
    const float inv = 1.0f / run_sum;
    T* orow = out + (size_t)token * n_head * v_dim + (size_t)head * v_dim;
    // an output gate: each feature times the logistic function of its gate value (32-bit)
    const T* grow = gate ? gate + (size_t)token * gate_stride + (size_t)head * v_dim : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) {
        const int d = lane + 32 * i;
        if (d < v_dim) {
            float o = acc[i] * inv;
            if (grow) o *= 1.0f / (1.0f + expf(-to_float(grow[d])));
            orow[d] = from_float<T>(o);
        }
    }
}

}  // namespace

// q: rows of `q_stride` elements whose first n_head * head_dim hold the queries; key pages
// [page, kv head, page_tokens, head_dim], value pages [page, kv head, page_tokens, v_dim] (keys and
// values may differ in size); block_table: [n_requests, max_pages]; out: [n_tokens, n_head * v_dim].
// gate (may be null): rows of `gate_stride` elements whose first n_head * v_dim hold gate values; the
// output is multiplied by their logistic function.  window <= 0: none.  slopes: [n_head] 32-bit or null;
// key_block <= 0: no block mask.  softcap > 0: a score s (scale included) becomes softcap * tanh(s / softcap)
// before the slopes and the softmax.  sinks: [n_head] 32-bit or null: exp(sink_h) is added to the softmax's
// denominator of head h (no key, no value; neither scaled nor capped).  v_stride: elements between the value
// rows of neighbouring tokens in `v_pages` (0: v_dim; larger where a token's values are the first v_dim
// features of a wider row, its key row for instance).
// num_pages: pages of the pool (with n_requests, what guarded builds hold the indices against).
MG_API int mg_paged_attention_general(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* token_request,
                                      const int* positions, void* out, int n_tokens, int n_head,
                                      int n_kv_head, int head_dim, int v_dim, const void* gate, int gate_stride,
                                      int page_tokens, int max_pages,
                                      int window, float scale, int num_pages, int n_requests, int is_bf16,
                                      const float* slopes, int key_block, float softcap, const float* sinks,
                                      int v_stride, void* stream) {
    if (n_tokens == 0) return MG_OK;
    if (v_stride <= 0) v_stride = v_dim;
    MG_REQUIRE(v_stride >= v_dim && softcap >= 0.f, "attention: bad value stride or cap");
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && page_tokens > 0 && max_pages > 0 && key_block >= 0,
               "attention: bad sizes");
    MG_REQUIRE(n_head % n_kv_head == 0, "attention: n_head %d is not a multiple of n_kv_head %d", n_head, n_kv_head);
    MG_REQUIRE(head_dim > 0 && head_dim <= MAX_KEY_DIM, "attention: head_dim %d is outside 1..%d", head_dim, MAX_KEY_DIM);
    MG_REQUIRE(v_dim > 0 && v_dim <= MAX_VALUE_DIM, "attention: value size %d is outside 1..%d", v_dim, MAX_VALUE_DIM);
    MG_REQUIRE(q_stride >= n_head * head_dim && (gate == nullptr || gate_stride >= n_head * v_dim),
               "attention: rows shorter than their heads");
    MG_REQUIRE(ceil_div(n_head, WARPS) <= 65535, "attention: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, ceil_div(n_head, WARPS)), block(32 * WARPS);
    const size_t smem = (size_t)WARPS * head_dim * sizeof(float);
#define MG_LAUNCH_GENERIC(T, DPL)                                                                                       \
    paged_attention_generic_kernel<T, DPL><<<grid, block, smem, s>>>(                                                   \
        (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table, token_request, positions, (T*)out,    \
        n_tokens, n_head, n_kv_head, head_dim, v_dim, (const T*)gate, gate_stride, page_tokens, max_pages, window,      \
        scale, num_pages, n_requests, slopes, key_block, softcap, sinks, v_stride)
    if (is_bf16) {
        if (v_dim <= 256) MG_LAUNCH_GENERIC(bf16, 8); else MG_LAUNCH_GENERIC(bf16, 16);
    } else {
        if (v_dim <= 256) MG_LAUNCH_GENERIC(float, 8); else MG_LAUNCH_GENERIC(float, 16);
    }
#undef MG_LAUNCH_GENERIC
    MG_CHECK_LAUNCH("paged_attention_generic");
    return MG_OK;
}

// The same for a fused projection's rows [q | k | v] with keys and values of one size:
// qkv: [n_tokens, (n_head + 2 n_kv_head) * head_dim]; out: [n_tokens, n_head * head_dim].
MG_API int mg_paged_attention_generic(const void* qkv, const void* k_pages, const void* v_pages,
                                      const int* block_table, const int* token_request,
                                      const int* positions, void* out, int n_tokens, int n_head,
                                      int n_kv_head, int head_dim, int page_tokens, int max_pages,
                                      int window, float scale, int num_pages, int n_requests, int is_bf16,
                                      void* stream) {
    return mg_paged_attention_general(qkv, (n_head + 2 * n_kv_head) * head_dim, k_pages, v_pages, block_table,
                                      token_request, positions, out, n_tokens, n_head, n_kv_head, head_dim, head_dim,
                                      nullptr, 0, page_tokens, max_pages, window, scale, num_pages, n_requests, is_bf16,
                                      nullptr, 0, 0.f, nullptr, 0, stream);
}
