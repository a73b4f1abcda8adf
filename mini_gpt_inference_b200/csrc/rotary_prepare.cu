// Between a fused projection and the attention, for mixers whose queries and keys turn with the position
// (rotary position encoding), one CTA per token:
//
// `qk_norm_rotary`: rows [ ... q (H x D) ... k (G x D) ... v (G x Dv) ... ].
//   * optionally one RMS norm over ALL query features of the token (H x D numbers at once, not head by head)
//     and one over all key features, each with a gain of that whole size;
//   * the first R features of every query and key head turn: feature i pairs with i + R/2,
//     (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * f_i, f_i given as a table of R/2 numbers;
//   * optionally every value head is divided by its root mean square (no gain), and optionally all its Dv features
//     turn with the position like a key head's would (feature m pairs with m + Dv/2, a = position * g_m, g_m given as
//     a second table of Dv/2 numbers): what attention then sums are values in the frame of their own positions;
//   * queries are written back in place, keys and values go to their cache rows.
//
// `rotate_heads`: rows [H x Dv] (the heads an attention over such values returns) turned by MINUS the token's own
// position, in place: the sum over the values comes back into the frame of the query.
//
// `latent_prepare`: rows [ ... q (H x (D + R)) ... low (C + R) ... ] of an attention whose keys and values are
// made from one small latent per token:
//   * the first C numbers of `low`, RMS-normed with a gain, are the latent; the last R turn with the position
//     and are one key part that all heads share; [latent | turned part] is the token's one cache row (and the
//     latent alone its value row, where values have pages of their own);
//   * the last R features of every query head turn the same way and are written to a second tensor, behind the
//     C numbers per head that a per-head product fills in: rows [H x (C + R)].
//
// Statistics, angles, sines and cosines are 32-bit: a = float(position) * f_i, then sincosf.  A token with a
// negative position (padding of a fixed-size batch) is skipped, a negative cache row is not written.
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(rotary_prepare)

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                                       // red may still be read from the call before
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) total += red[w];
    return total;
}

// the value of feature d of a head after the turn; `head` points at the head's features in shared memory
__device__ __forceinline__ float turned(const float* head, const float* gain, float r, int d, int rot, const float* cs) {
    const float x = gain ? head[d] * r * gain[d] : head[d] * r;
    if (d >= rot) return x;
    const int half = rot >> 1;
    const int i = d < half ? d : d - half, partner = d < half ? d + half : d - half;
    const float y = gain ? head[partner] * r * gain[partner] : head[partner] * r;
    const float c = cs[2 * i], s = cs[2 * i + 1];
    return d < half ? x * c - y * s : x * c + y * s;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
qk_norm_rotary_kernel(T* __restrict__ proj, int ld, int n_head, int n_kv_head, int head_dim, int v_dim, int q_off,
                      int k_off, int v_off, int norm, float eps, const float* __restrict__ q_gain,
                      const float* __restrict__ k_gain, int rot, const float* __restrict__ freq,
                      const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, int page_tokens, int num_pages, int v_norm, float v_eps,
                      const float* __restrict__ v_freq) {
    extern __shared__ float smem[];                        // [H*D] q, [G*D] k, [rot] cos/sin pairs
    __shared__ float red[THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[token];
    if (pos < 0) return;
    const int qn = n_head * head_dim, kn = n_kv_head * head_dim;
    float* qs = smem;
    float* ks = qs + qn;
    float* cs = ks + kn;
    T* row = proj + (size_t)token * ld;
    float sq_q = 0.f, sq_k = 0.f;
    for (int i = tid; i < qn; i += THREADS) {
        const float x = to_float(row[q_off + i]);
        qs[i] = x;
        sq_q = fmaf(x, x, sq_q);
    }
    for (int i = tid; i < kn; i += THREADS) {
        const float x = to_float(row[k_off + i]);
        ks[i] = x;
        sq_k = fmaf(x, x, sq_k);
    }
    for (int i = tid; i < rot / 2; i += THREADS) {
        const float a = __fmul_rn((float)pos, freq[i]);
        float s, c;
        sincosf(a, &s, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = s;
    }
    float rq = 1.f, rk = 1.f;
    if (norm) {
        rq = 1.0f / sqrtf(block_sum(sq_q, red) / (float)qn + eps);
        rk = 1.0f / sqrtf(block_sum(sq_k, red) / (float)kn + eps);
    } else {
        __syncthreads();
    }
    for (int i = tid; i < qn; i += THREADS) {
        const int h = i / head_dim, d = i - h * head_dim;
        row[q_off + i] = from_float<T>(turned(qs + h * head_dim, q_gain ? q_gain + h * head_dim : nullptr, rq, d, rot, cs));
    }
    int slot = slots ? slots[token] : -1;
    if (slot >= 0 && !MG_GUARDED(rotary_prepare, MG_GUARD_CACHE_ROW, slot, (long long)num_pages * page_tokens)) slot = -1;
    if (k_pages == nullptr || slot < 0) return;
    const int page = slot / page_tokens, within = slot - page * page_tokens;
    for (int i = tid; i < kn; i += THREADS) {
        const int h = i / head_dim, d = i - h * head_dim;
        k_pages[(((size_t)page * n_kv_head + h) * page_tokens + within) * head_dim + d] =
            from_float<T>(turned(ks + h * head_dim, k_gain ? k_gain + h * head_dim : nullptr, rk, d, rot, cs));
    }
    if (!v_norm && v_freq == nullptr) {
        for (int i = tid; i < n_kv_head * v_dim; i += THREADS) {
            const int h = i / v_dim, d = i - h * v_dim;
            v_pages[(((size_t)page * n_kv_head + h) * page_tokens + within) * v_dim + d] = row[v_off + i];
        }
        return;
    }
    // a warp takes a value head at a time: its root mean square, then the turn of all its features
    const int warp = tid >> 5, lane = tid & 31, half = v_dim >> 1;
    for (int h = warp; h < n_kv_head; h += THREADS / 32) {
        const T* src = row + v_off + (size_t)h * v_dim;
        T* dst = v_pages + (((size_t)page * n_kv_head + h) * page_tokens + within) * v_dim;
        float r = 1.f;
        if (v_norm) {
            float sq = 0.f;
            for (int d = lane; d < v_dim; d += 32) {
                const float x = to_float(src[d]);
                sq = fmaf(x, x, sq);
            }
            r = 1.0f / sqrtf(warp_sum(sq) / (float)v_dim + v_eps);
        }
        if (v_freq == nullptr) {
            for (int d = lane; d < v_dim; d += 32) dst[d] = from_float<T>(to_float(src[d]) * r);
            continue;
        }
        for (int m = lane; m < half; m += 32) {
            float sn, cs2;
            sincosf(__fmul_rn((float)pos, v_freq[m]), &sn, &cs2);
            const float u = to_float(src[m]) * r, v = to_float(src[m + half]) * r;
            dst[m] = from_float<T>(u * cs2 - v * sn);
            dst[m + half] = from_float<T>(v * cs2 + u * sn);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
rotate_heads_kernel(T* __restrict__ x, int n_head, int v_dim, const float* __restrict__ freq,
                    const int* __restrict__ positions, float sign) {
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, half = v_dim >> 1;
    const int pos = positions[token];
    if (pos < 0) return;
    T* row = x + (size_t)token * n_head * v_dim;
    for (int i = threadIdx.x; i < n_head * half; i += THREADS) {
        const int h = i / half, m = i - h * half;
        float sn, cs;
        sincosf(__fmul_rn((float)pos, freq[m]), &sn, &cs);
        sn *= sign;
        T* head = row + (size_t)h * v_dim;
        const float u = to_float(head[m]), v = to_float(head[m + half]);
        head[m] = from_float<T>(u * cs - v * sn);
        head[m + half] = from_float<T>(v * cs + u * sn);
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
latent_prepare_kernel(const T* __restrict__ proj, int ld, int n_head, int q_off, int q_dim, int rot, int low_off, int rank,
                      const float* __restrict__ gain, float eps, const float* __restrict__ freq, T* __restrict__ q_out,
                      const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, int page_tokens, int num_pages) {
    extern __shared__ float smem[];                        // [rank + rot] low, [rot] cos/sin pairs
    __shared__ float red[THREADS / 32];
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[token];
    if (pos < 0) return;
    float* low = smem;
    float* cs = low + rank + rot;
    const T* row = proj + (size_t)token * ld;
    const int half = rot >> 1;
    for (int i = tid; i < half; i += THREADS) {
        const float a = __fmul_rn((float)pos, freq[i]);
        float s, c;
        sincosf(a, &s, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = s;
    }
    int slot = slots ? slots[token] : -1;
    if (slot >= 0 && !MG_GUARDED(rotary_prepare, MG_GUARD_CACHE_ROW, slot, (long long)num_pages * page_tokens)) slot = -1;
    const bool store = k_pages != nullptr && slot >= 0;    // (a layer that reads another layer's latents stores none)
    float sq = 0.f;
    if (store) {
        for (int i = tid; i < rank + rot; i += THREADS) {
            const float x = to_float(row[low_off + i]);
            low[i] = x;
            if (i < rank) sq = fmaf(x, x, sq);
        }
    }
    const float total = block_sum(sq, red);                // (also the barrier behind cs and low)
    // the turning part of every query head, behind the room for the head's latent-sized part
    const int out_head = rank + rot;
    for (int i = tid; i < n_head * rot; i += THREADS) {
        const int h = i / rot, d = i - h * rot;
        const T* qh = row + q_off + (size_t)h * (q_dim + rot) + q_dim;
        const int j = d < half ? d : d - half;
        const float x = to_float(qh[d]), y = to_float(qh[d < half ? d + half : d - half]);
        const float c = cs[2 * j], s = cs[2 * j + 1];
        q_out[((size_t)token * n_head + h) * out_head + rank + d] = from_float<T>(d < half ? x * c - y * s : x * c + y * s);
    }
    if (!store) return;
    const float r = 1.0f / sqrtf(total / (float)rank + eps);
    const int page = slot / page_tokens, within = slot - page * page_tokens;
    T* krow = k_pages + ((size_t)page * page_tokens + within) * out_head;
    T* vrow = v_pages ? v_pages + ((size_t)page * page_tokens + within) * rank : nullptr;
    for (int i = tid; i < rank; i += THREADS) {
        const T c = from_float<T>(low[i] * r * gain[i]);
        krow[i] = c;
        if (vrow) vrow[i] = c;
    }
    for (int d = tid; d < rot; d += THREADS) {
        const int j = d < half ? d : d - half;
        const float x = low[rank + d], y = low[rank + (d < half ? d + half : d - half)];
        const float c = cs[2 * j], s = cs[2 * j + 1];
        krow[rank + d] = from_float<T>(d < half ? x * c - y * s : x * c + y * s);
    }
}

}  // namespace

// proj: [n_tokens, ld] rows (bfloat16 if is_bf16 else 32-bit), queries rewritten in place; q_gain: [n_head *
// head_dim], k_gain: [n_kv_head * head_dim] 32-bit (used if norm; either may be null: no gain); rot: features of
// a head that turn (even, <= head_dim; 0: none); freq: [rot / 2] 32-bit on the device; positions: [n_tokens];
// slots: [n_tokens] flat cache rows or null with the pages (nothing is cached); key pages [page, kv head,
// page_tokens, head_dim], value pages [page, kv head, page_tokens, v_dim].
MG_API int mg_qk_norm_rotary(void* proj, int ld, int n_tokens, int n_head, int n_kv_head, int head_dim, int v_dim, int q_off,
                             int k_off, int v_off, int norm, float eps, const float* q_gain, const float* k_gain, int rot,
                             const float* freq, const int* positions, const int* slots, void* k_pages, void* v_pages,
                             int page_tokens, int num_pages, int is_bf16, int v_norm, float v_eps, const float* v_freq,
                             void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(v_freq == nullptr || v_dim % 2 == 0, "qk_norm_rotary: value heads of %d features do not turn in pairs", v_dim);
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && head_dim > 0 && v_dim > 0 && positions != nullptr,
               "qk_norm_rotary: bad sizes");
    MG_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= head_dim && (rot == 0 || freq != nullptr),
               "qk_norm_rotary: %d turning features in heads of %d", rot, head_dim);
    MG_REQUIRE(q_off >= 0 && k_off >= 0 && v_off >= 0 && q_off + n_head * head_dim <= ld &&
                   k_off + n_kv_head * head_dim <= ld && v_off + n_kv_head * v_dim <= ld,
               "qk_norm_rotary: heads outside the rows");
    MG_REQUIRE((k_pages == nullptr) == (v_pages == nullptr) && (k_pages == nullptr || (slots && page_tokens > 0)),
               "qk_norm_rotary: pages without cache rows");
    const size_t smem = sizeof(float) * ((size_t)(n_head + n_kv_head) * head_dim + rot);
    MG_REQUIRE(smem <= 160 * 1024, "qk_norm_rotary: a token's queries and keys do not fit shared memory");
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (is_bf16) {
        e = smem > 48 * 1024 ? cudaFuncSetAttribute(qk_norm_rotary_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) : cudaSuccess;
        if (e == cudaSuccess)
            e = mg_launch(qk_norm_rotary_kernel<bf16>, dim3(n_tokens), dim3(THREADS), smem, s, true, (bf16*)proj, ld, n_head,
                          n_kv_head, head_dim, v_dim, q_off, k_off, v_off, norm, eps, q_gain, k_gain, rot, freq, positions,
                          slots, (bf16*)k_pages, (bf16*)v_pages, page_tokens, num_pages, v_norm, v_eps, v_freq);
    } else {
        e = smem > 48 * 1024 ? cudaFuncSetAttribute(qk_norm_rotary_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) : cudaSuccess;
        if (e == cudaSuccess)
            e = mg_launch(qk_norm_rotary_kernel<float>, dim3(n_tokens), dim3(THREADS), smem, s, true, (float*)proj, ld, n_head,
                          n_kv_head, head_dim, v_dim, q_off, k_off, v_off, norm, eps, q_gain, k_gain, rot, freq, positions,
                          slots, (float*)k_pages, (float*)v_pages, page_tokens, num_pages, v_norm, v_eps, v_freq);
    }
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "qk_norm_rotary: %s", cudaGetErrorString(e));
    return MG_OK;
}

// x: [n_tokens, n_head * v_dim], in place; freq: [v_dim / 2] 32-bit; sign: -1 turns back, +1 forward.
MG_API int mg_rotate_heads(void* x, int n_tokens, int n_head, int v_dim, const float* freq, const int* positions,
                           float sign, int is_bf16, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && v_dim > 0 && v_dim % 2 == 0 && freq && positions, "rotate_heads: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const cudaError_t e =
        is_bf16 ? mg_launch(rotate_heads_kernel<bf16>, dim3(n_tokens), dim3(THREADS), 0, s, true, (bf16*)x, n_head, v_dim,
                            freq, positions, sign)
                : mg_launch(rotate_heads_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, s, true, (float*)x, n_head, v_dim,
                            freq, positions, sign);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "rotate_heads: %s", cudaGetErrorString(e));
    return MG_OK;
}

// proj: [n_tokens, ld] rows holding the query heads (n_head x (q_dim + rot) from q_off) and, if the layer makes
// latents of its own (k_pages not null), `low` (rank + rot numbers from low_off); gain: [rank] 32-bit; freq:
// [rot / 2]; q_out: [n_tokens, n_head * (rank + rot)], of which the last rot of every head are written; key pages
// [page, 1, page_tokens, rank + rot]; value pages [page, 1, page_tokens, rank] or null (values read from the key
// rows).
MG_API int mg_latent_prepare(const void* proj, int ld, int n_tokens, int n_head, int q_off, int q_dim, int rot, int low_off,
                             int rank, const float* gain, float eps, const float* freq, void* q_out, const int* positions,
                             const int* slots, void* k_pages, void* v_pages, int page_tokens, int num_pages, int is_bf16,
                             void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && q_dim > 0 && rank > 0 && positions != nullptr && q_out != nullptr,
               "latent_prepare: bad sizes");
    MG_REQUIRE(rot >= 0 && rot % 2 == 0 && (rot == 0 || freq != nullptr), "latent_prepare: %d turning features", rot);
    MG_REQUIRE(q_off >= 0 && q_off + n_head * (q_dim + rot) <= ld, "latent_prepare: queries outside the rows");
    MG_REQUIRE(k_pages == nullptr || (slots && page_tokens > 0 && gain && low_off >= 0 && low_off + rank + rot <= ld),
               "latent_prepare: pages without cache rows, a gain or the rows' latent part");
    MG_REQUIRE(k_pages != nullptr || v_pages == nullptr, "latent_prepare: value pages without key pages");
    const size_t smem = sizeof(float) * ((size_t)rank + 2 * rot);
    MG_REQUIRE(smem <= 160 * 1024, "latent_prepare: a latent of %d numbers does not fit shared memory", rank);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (is_bf16) {
        e = smem > 48 * 1024 ? cudaFuncSetAttribute(latent_prepare_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) : cudaSuccess;
        if (e == cudaSuccess)
            e = mg_launch(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(THREADS), smem, s, true, (const bf16*)proj, ld,
                          n_head, q_off, q_dim, rot, low_off, rank, gain, eps, freq, (bf16*)q_out, positions, slots,
                          (bf16*)k_pages, (bf16*)v_pages, page_tokens, num_pages);
    } else {
        e = smem > 48 * 1024 ? cudaFuncSetAttribute(latent_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) : cudaSuccess;
        if (e == cudaSuccess)
            e = mg_launch(latent_prepare_kernel<float>, dim3(n_tokens), dim3(THREADS), smem, s, true, (const float*)proj, ld,
                          n_head, q_off, q_dim, rot, low_off, rank, gain, eps, freq, (float*)q_out, positions, slots,
                          (float*)k_pages, (float*)v_pages, page_tokens, num_pages);
    }
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "latent_prepare: %s", cudaGetErrorString(e));
    return MG_OK;
}
