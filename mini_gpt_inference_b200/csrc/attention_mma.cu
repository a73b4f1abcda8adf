// Causal attention over the paged cache on the warp-level tensor cores, for key and value heads of
// different sizes, grouped query heads, a window and an output gate; bfloat16 in, 32-bit softmax.
//
// The rows of a tile are (token, query head of one key/value head's group) pairs; a CTA of four warps
// walks blocks of 64 keys: keys and values of the block come from their pages into padded shared
// memory (cp.async, two buffers in turn), S = Q K^T by mma.sync m16n8k16 (Q fragments stay in registers), the running maximum, sum
// and the weights in 32-bit, P rounded to bfloat16 as the A operand of O += P V (V through
// ldmatrix.trans).  Head sizes are rounded up to a compiled size (64, 96 or 128 key features, 64 or
// 128 value features); the padding is zeros in registers and shared memory.
//
//   tiles  (portions of prompts): a tile is 64 / group consecutive tokens of one request with all the
//          group's heads, 16 rows per warp; every warp walks every key block.  The CTA finds its
//          request and tile from the requests' token counts on the device.
//   split  (single tokens): a CTA is one token, one key/value head and one range of keys; the
//          (128 keys unless the longest possible context would need more than 1,024 ranges); the
//          group's heads are the rows of one m16 tile, each warp takes 16 of a block's 64 keys, the
//          warps' partial results meet in shared memory and go to scratch; the CTA that finishes a
//          (token, key/value head) last merges the ranges, applies the gate and stores (or a second
//          kernel does, if no counters are given).
//
// Further, all parameters: `softcap` (a score s, scale included, becomes softcap * tanh(s / softcap)), `sinks`
// (one learned number per head whose exponential joins the softmax's denominator, with no key and no value: it is
// added where a row's sum is final, in the tiles' epilogue and in the merge of the ranges), and `v_stride` (a
// token's values are the first dv features of a wider row, its key row for instance).
//
// Keys are always read from the pages, whichever step wrote them.  Rows of pages beyond a request's
// last key are never multiplied into a result (their values are replaced by zeros in shared memory).
#include <math.h>

#include "common.cuh"

MG_GUARD_DECLARE(attention_mma)

namespace {

constexpr int KB = 64;            // keys per block
constexpr int PAD = 8;            // bfloat16 elements of padding per shared-memory row
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
    const bf16* q;                // rows of q_stride elements, heads of D
    int q_stride;
    const bf16* k_pages;          // [page, G, page_tokens, D]
    const bf16* v_pages;          // [page, G, page_tokens, DV]
    const int* block_table;       // [n_requests, max_pages]
    const int* token_request;     // [n_tokens]
    const int* positions;         // [n_tokens]
    const int* req_q_start;       // [n_requests]
    const int* req_q_len;         // [n_requests]
    const bf16* gate;             // rows of gate_stride elements, heads of DV; may be null
    int gate_stride;
    bf16* out;                    // [n_tokens, H * DV]
    float* part_o;                // split: [n_tokens, H, splits, DV]
    float* part_ml;               // split: [n_tokens, H, splits, 2]
    int* counters;                // split: [n_tokens, G] zeros, left as zeros (null: a second kernel merges)
    int n_tokens, n_requests, n_head, n_kv_head, d, dv, page_tokens, max_pages, window, num_pages;
    int tile_tokens;              // tiles: tokens per tile
    int splits, split_keys;       // split: ranges of keys per token
    float scale_log2;             // scale * log2(e)
    const float* slopes;          // [H] or null: slope_h * (i - j) is taken off the score of query i and key j
    int block;                    // > 0: a query sees only the keys of its own block of this many positions
    float cap_log2;               // > 0: softcap * log2(e)
    const float* sinks;           // [H] or null
    int v_stride;                 // elements between the value rows of neighbouring tokens
};

// What a head's sink adds to a row's sum that is held relative to the maximum m (in powers of two).
__device__ __forceinline__ float sink_term(const AttnParams& p, int head, float m) {
    return p.sinks ? exp2f(p.sinks[head] * LOG2E - m) : 0.f;
}

// The first key that a query at `pos` sees: the window's, raised to the first position of the query's block.
__device__ __forceinline__ int first_visible(const AttnParams& p, int pos) {
    int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    if (p.block > 0) lo = max(lo, pos / p.block * p.block);
    return lo;
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Keys j0 .. j0+63 of one request and key/value head into shared memory, asynchronously: rows
// [KB][DP+PAD] and [KB][DVP+PAD].  Rows outside lo..hi become zeros (they may hold anything in the
// pages).  The caller commits the group and waits for it.
__device__ __forceinline__ void cp_async16(bf16* dst, const bf16* src, bool real) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = real ? 16 : 0;                       // 0: nothing is read, the 16 bytes become zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A warp copies 16 of the block's 64 rows; a row's 16-byte chunks (keys first, then values) go to
// neighbouring lanes, 8, 16 or 32 lanes per row, so no division sits in the loop (page sizes that
// are powers of two index their pages by shifts: page_shift >= 0).
template <int DP, int DVP>
__device__ __forceinline__ void load_block(const AttnParams& p, const int* table, int kv_head, int j0, int lo, int hi,
                                           bf16* ks, bf16* vs, int warp, int lane, int page_shift) {
    const int kc = p.d >> 3, chunks = kc + (p.dv >> 3);  // 16-byte chunks per row, at most 32
    const int lane_shift = chunks <= 8 ? 3 : chunks <= 16 ? 4 : 5;
    const int c = lane & ((1 << lane_shift) - 1);
    for (int key = warp * 16 + (lane >> lane_shift); key < warp * 16 + 16; key += 32 >> lane_shift) {
        if (c >= chunks) continue;
        const int j = j0 + key;
        const bool real = j >= lo && j <= hi;
        size_t row = 0;
        if (real) {
            const int index = page_shift >= 0 ? j >> page_shift : j / p.page_tokens;
            const int within = page_shift >= 0 ? j & (p.page_tokens - 1) : j - index * p.page_tokens;
            int page = table[index];
            if (!MG_GUARDED(attention_mma, MG_GUARD_PAGE, page, p.num_pages)) page = 0;
            row = ((size_t)page * p.n_kv_head + kv_head) * p.page_tokens + within;
        }
        if (c < kc) cp_async16(ks + key * (DP + PAD) + c * 8, p.k_pages + row * p.d + c * 8, real);
        else cp_async16(vs + key * (DVP + PAD) + (c - kc) * 8, p.v_pages + row * p.v_stride + (c - kc) * 8, real);
    }
}

// Zero the columns that the loads never write (head sizes below the compiled ones).
template <int DP, int DVP>
__device__ __forceinline__ void zero_padding(const AttnParams& p, bf16* ks, bf16* vs, int tid, int threads) {
    const bf16 z = __float2bfloat16_rn(0.f);
    if (p.d < DP)
        for (int i = tid; i < KB * (DP - p.d); i += threads) ks[(i / (DP - p.d)) * (DP + PAD) + p.d + i % (DP - p.d)] = z;
    if (p.dv < DVP)
        for (int i = tid; i < KB * (DVP - p.dv); i += threads) vs[(i / (DVP - p.dv)) * (DVP + PAD) + p.dv + i % (DVP - p.dv)] = z;
}

// The query fragments of a lane's two rows (null pointer: zeros), columns beyond d as zeros.
template <int DP>
__device__ __forceinline__ void load_q(uint32_t (&qf)[DP / 16][4], const bf16* q0, const bf16* q1, int d, int lane) {
    const int c = 2 * (lane & 3);
#pragma unroll
    for (int ks = 0; ks < DP / 16; ++ks) {
        const int c0 = 16 * ks + c, c1 = c0 + 8;
        qf[ks][0] = (q0 && c0 < d) ? *reinterpret_cast<const uint32_t*>(q0 + c0) : 0u;
        qf[ks][1] = (q1 && c0 < d) ? *reinterpret_cast<const uint32_t*>(q1 + c0) : 0u;
        qf[ks][2] = (q0 && c1 < d) ? *reinterpret_cast<const uint32_t*>(q0 + c1) : 0u;
        qf[ks][3] = (q1 && c1 < d) ? *reinterpret_cast<const uint32_t*>(q1 + c1) : 0u;
    }
}

// One warp, its 16 rows, NT * 8 keys of the block in shared memory starting at key `k_first`:
// scores, masks, the running maximum and sum, and O += P V.  pos/lo: the two rows' own last and first
// visible key (pos < 0: a row without a token).
template <int DP, int DVP, int NT>
__device__ __forceinline__ void attend(const uint32_t (&qf)[DP / 16][4], const bf16* ks, const bf16* vs, int k_first,
                                       int j_first, const int (&pos)[2], const int (&lo)[2], bool all_visible,
                                       float scale_log2, float (&m)[2], float (&l)[2], float (&o)[DVP / 8][4], int lane,
                                       const float (&slope_log2)[2], bool biased, float cap_log2) {
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b[4];
            ldsm4(b, ks + (k_first + n * 8 + (lane >> 4) * 8 + (lane & 7)) * (DP + PAD) + kk * 16 + ((lane >> 3) & 1) * 8);
            mma16816(s[n], qf[kk], b[0], b[1]);
            mma16816(s[n + 1], qf[kk], b[2], b[3]);
        }
    }
    // masks and the block's maximum per row (all_visible, the same for the whole warp: every row of
    // the warp sees every key of these, nothing to compare)
    float bm[2] = {-INFINITY, -INFINITY};
    if (all_visible && !biased) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[n][e] *= scale_log2;
                bm[e >> 1] = fmaxf(bm[e >> 1], s[n][e]);
            }
    } else if (biased) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j_first + n * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
                float sc = s[n][e] * scale_log2;
                if (cap_log2 > 0.f) sc = cap_log2 * tanhf(sc / cap_log2);
                const float v = (j <= pos[r] && j >= lo[r]) ? sc - slope_log2[r] * (float)(pos[r] - j) : -INFINITY;
                s[n][e] = v;
                bm[r] = fmaxf(bm[r], v);
            }
    } else {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j_first + n * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
                const float v = (j <= pos[r] && j >= lo[r]) ? s[n][e] * scale_log2 : -INFINITY;
                s[n][e] = v;
                bm[r] = fmaxf(bm[r], v);
            }
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 1));
        bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 2));
        const float nm = fmaxf(m[r], bm[r]);
        corr[r] = (m[r] == -INFINITY) ? 0.f : exp2_approx(m[r] - nm);
        base[r] = (nm == -INFINITY) ? 0.f : nm;            // a row that has seen no key yet: weights stay 0
        m[r] = nm;
    }
    float bs[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pr = exp2_approx(s[n][e] - base[e >> 1]);
            s[n][e] = pr;
            bs[e >> 1] += pr;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        bs[r] += __shfl_xor_sync(0xffffffffu, bs[r], 1);
        bs[r] += __shfl_xor_sync(0xffffffffu, bs[r], 2);
        l[r] = l[r] * corr[r] + bs[r];
    }
#pragma unroll
    for (int n = 0; n < DVP / 8; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
    }
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {                  // 16 keys at a time
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n = 0; n < DVP / 8; n += 2) {
            uint32_t b[4];
            ldsm4_t(b, vs + (k_first + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * (DVP + PAD) + n * 8 + (lane >> 4) * 8);
            mma16816(o[n], a, b[0], b[1]);
            mma16816(o[n + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ float logistic(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- portions of prompts ---------------------------------------------------------------------------
template <int DP, int DVP>
__global__ void __launch_bounds__(128, (DP + DVP <= 160) ? 3 : ((DP + DVP <= 192) ? 2 : 1))
attention_tiles_kernel(const AttnParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int STAGE = KB * (DP + PAD + DVP + PAD);     // elements of one buffer: keys, then values
    bf16* ks = reinterpret_cast<bf16*>(smem_raw);
    bf16* vs = ks + KB * (DP + PAD);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    zero_padding<DP, DVP>(p, ks, vs, tid, 128);
    zero_padding<DP, DVP>(p, ks + STAGE, vs + STAGE, tid, 128);
    pdl_trigger();
    pdl_wait();
    // which request, which tile of it; the grid's first CTAs take the last tiles, whose tokens see the
    // most keys, so that the long ones do not start last
    int tile = (int)(gridDim.x - 1 - blockIdx.x), request = 0;
    for (; request < p.n_requests; ++request) {
        const int tiles = (p.req_q_len[request] + p.tile_tokens - 1) / p.tile_tokens;
        if (tile < tiles) break;
        tile -= tiles;
    }
    if (request >= p.n_requests) return;
    const int kv_head = blockIdx.y, group = p.n_head / p.n_kv_head;
    const int first = p.req_q_start[request] + tile * p.tile_tokens;
    const int count = min(p.tile_tokens, p.req_q_len[request] - tile * p.tile_tokens);
    int hi = p.positions[first + count - 1], lo_tile = 0;
    if (hi < 0) return;                                     // padding
    if (!MG_GUARDED(attention_mma, MG_GUARD_POSITION, hi, (long long)p.max_pages * p.page_tokens)) hi = 0;
    if (p.window > 0 || p.block > 0) lo_tile = first_visible(p, max(0, p.positions[first]));
    const int* table = p.block_table + (size_t)request * p.max_pages;

    // this lane's two rows
    int pos[2], lo[2], token[2], head[2];
    const bf16* qrow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + 8 * r;
        const int t = row / group;
        const bool live = t < count;
        token[r] = first + (live ? t : 0);
        head[r] = kv_head * group + row % group;
        pos[r] = live ? p.positions[token[r]] : -1;
        lo[r] = pos[r] >= 0 ? first_visible(p, pos[r]) : 0;
        qrow[r] = live ? p.q + (size_t)token[r] * p.q_stride + (size_t)head[r] * p.d : nullptr;
    }
    const bool biased = p.slopes != nullptr || p.cap_log2 > 0.f;
    const float slope_log2[2] = {p.slopes ? p.slopes[head[0]] * LOG2E : 0.f, p.slopes ? p.slopes[head[1]] * LOG2E : 0.f};
    uint32_t qf[DP / 16][4];
    load_q<DP>(qf, qrow[0], qrow[1], p.d, lane);
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[DVP / 8][4];
#pragma unroll
    for (int n = 0; n < DVP / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    // the last key this warp's rows can see (rows are in token order)
    const int warp_last_token = min(count - 1, (warp * 16 + 15) / group);
    const int warp_hi = (warp * 16) / group < count ? p.positions[first + warp_last_token] : -1;
    // blocks that all rows of the warp see whole: up to the warp's first token, from the last one's window on
    const int warp_first_pos = (warp * 16) / group < count ? p.positions[first + (warp * 16) / group] : -1;
    const int warp_max_lo = warp_hi >= 0 ? first_visible(p, warp_hi) : 0;

    // two buffers take turns: the next block's copies are in flight while this one is multiplied
    const int j_begin = (lo_tile / KB) * KB;
    const int page_shift = (p.page_tokens & (p.page_tokens - 1)) == 0 ? __ffs(p.page_tokens) - 1 : -1;
    load_block<DP, DVP>(p, table, kv_head, j_begin, lo_tile, hi, ks, vs, warp, lane, page_shift);
    cp_async_commit();
    int buf = 0;
    for (int j0 = j_begin; j0 <= hi; j0 += KB, buf ^= 1) {
        if (j0 + KB <= hi) {
            load_block<DP, DVP>(p, table, kv_head, j0 + KB, lo_tile, hi, ks + (buf ^ 1) * STAGE, vs + (buf ^ 1) * STAGE, warp, lane,
                                page_shift);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j0 <= warp_hi)
            attend<DP, DVP, 8>(qf, ks + buf * STAGE, vs + buf * STAGE, 0, j0, pos, lo,
                               j0 + KB - 1 <= warp_first_pos && j0 >= warp_max_lo, p.scale_log2, m, l, o, lane, slope_log2,
                               biased, p.cap_log2);
        __syncthreads();                                    // the buffer is free for the block after the next
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (pos[r] < 0) continue;
        l[r] += sink_term(p, head[r], m[r]);
        const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
        bf16* orow = p.out + (size_t)token[r] * p.n_head * p.dv + (size_t)head[r] * p.dv;
        const bf16* grow = p.gate ? p.gate + (size_t)token[r] * p.gate_stride + (size_t)head[r] * p.dv : nullptr;
#pragma unroll
        for (int n = 0; n < DVP / 8; ++n) {
            const int c = n * 8 + 2 * (lane & 3);
            if (c >= p.dv) continue;
            float a = o[n][2 * r] * inv, b = o[n][2 * r + 1] * inv;
            if (grow) {
                const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(grow + c);
                a *= logistic(__bfloat162float(g.x));
                b *= logistic(__bfloat162float(g.y));
            }
            *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16(a, b);
        }
    }
}

// ---- single tokens, the keys cut into ranges ---------------------------------------------------------
template <int DP, int DVP>
__global__ void __launch_bounds__(128)
attention_split_kernel(const AttnParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr int STAGE = KB * (DP + PAD + DVP + PAD);     // elements of one buffer: keys, then values
    bf16* ks = reinterpret_cast<bf16*>(smem_raw);
    bf16* vs = ks + KB * (DP + PAD);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    zero_padding<DP, DVP>(p, ks, vs, tid, 128);
    zero_padding<DP, DVP>(p, ks + STAGE, vs + STAGE, tid, 128);
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, kv_head = blockIdx.y, split = blockIdx.z;
    const int group = p.n_head / p.n_kv_head;
    int position = p.positions[token];
    const bool padding = position < 0;
    if (!padding && !MG_GUARDED(attention_mma, MG_GUARD_POSITION, position, (long long)p.max_pages * p.page_tokens)) position = 0;
    const int lo_row = padding ? 0 : first_visible(p, position);
    const int first = (lo_row / KB) * KB + split * p.split_keys;         // ranges start at the window's block
    const int last = min(position, first + p.split_keys - 1);
    // ranges that hold keys of this token; the others have nothing to do (the grid is sized for the
    // longest context there can be)
    const int live = padding ? 0 : (position - (lo_row / KB) * KB) / p.split_keys + 1;
    if (split >= live) {
        if (padding && split == 0)                                        // a padding row's output is zeros
            for (int i = tid; i < group * p.dv; i += 128)
                p.out[(size_t)token * p.n_head * p.dv + (size_t)kv_head * group * p.dv + i] = __float2bfloat16_rn(0.f);
        return;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[DVP / 8][4];
#pragma unroll
    for (int n = 0; n < DVP / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const int row0 = lane >> 2;                              // rows are the group's heads; row0 + 8 as well
    if (!padding && first <= last) {
        int request = p.token_request[token];
        if (!MG_GUARDED(attention_mma, MG_GUARD_REQUEST, request, p.n_requests)) request = 0;
        const int* table = p.block_table + (size_t)request * p.max_pages;
        int pos[2], lo[2];
        const bf16* qrow[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = row0 + 8 * r;
            const bool has_row = row < group;
            pos[r] = has_row ? position : -1;
            lo[r] = lo_row;
            qrow[r] = has_row ? p.q + (size_t)token * p.q_stride + (size_t)(kv_head * group + row) * p.d : nullptr;
        }
        const bool biased = p.slopes != nullptr || p.cap_log2 > 0.f;
        const float slope_log2[2] = {p.slopes && row0 < group ? p.slopes[kv_head * group + row0] * LOG2E : 0.f,
                                     p.slopes && row0 + 8 < group ? p.slopes[kv_head * group + row0 + 8] * LOG2E : 0.f};
        uint32_t qf[DP / 16][4];
        load_q<DP>(qf, qrow[0], qrow[1], p.d, lane);
        const int page_shift = (p.page_tokens & (p.page_tokens - 1)) == 0 ? __ffs(p.page_tokens) - 1 : -1;
        load_block<DP, DVP>(p, table, kv_head, first, lo_row, last, ks, vs, warp, lane, page_shift);
        cp_async_commit();
        int buf = 0;
        for (int j0 = first; j0 <= last; j0 += KB, buf ^= 1) {
            if (j0 + KB <= last) {
                load_block<DP, DVP>(p, table, kv_head, j0 + KB, lo_row, last, ks + (buf ^ 1) * STAGE, vs + (buf ^ 1) * STAGE, warp,
                                    lane, page_shift);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            if (j0 + warp * 16 <= last)
                attend<DP, DVP, 2>(qf, ks + buf * STAGE, vs + buf * STAGE, warp * 16, j0 + warp * 16, pos, lo, false,
                                   p.scale_log2, m, l, o, lane, slope_log2, biased, p.cap_log2);
            __syncthreads();
        }
    }
    // the four warps' partial results meet in shared memory (after the last block has been used)
    __syncthreads();
    float* sm_ml = reinterpret_cast<float*>(smem_raw);               // [4][16][2]
    float* sm_o = sm_ml + 4 * 16 * 2;                                 // [4][16][DVP]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + 8 * r;
        if ((lane & 3) == 0) {
            sm_ml[(warp * 16 + row) * 2] = m[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l[r];
        }
#pragma unroll
        for (int n = 0; n < DVP / 8; ++n) {
            const int c = n * 8 + 2 * (lane & 3);
            sm_o[(warp * 16 + row) * DVP + c] = o[n][2 * r];
            sm_o[(warp * 16 + row) * DVP + c + 1] = o[n][2 * r + 1];
        }
    }
    __syncthreads();
    for (int i = tid; i < group * p.dv; i += 128) {
        const int row = i / p.dv, c = i - row * p.dv;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_ml[(w * 16 + row) * 2]);
        float sum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_ml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            sum += f * sm_ml[(w * 16 + row) * 2 + 1];
            acc += f * sm_o[(w * 16 + row) * DVP + c];
        }
        const size_t slot = ((size_t)token * p.n_head + kv_head * group + row) * p.splits + split;
        p.part_o[slot * p.dv + c] = acc;
        if (c == 0) {
            p.part_ml[slot * 2] = mm;
            p.part_ml[slot * 2 + 1] = sum;
        }
    }
    if (p.counters == nullptr) return;
    // The CTA that finishes a (token, key/value head) last merges its ranges: an arrive-only counter,
    // nobody waits.  It leaves the counter at zero for the next launch.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = p.counters + (size_t)token * p.n_kv_head + kv_head;
        is_last = atomicAdd(counter, 1) == live - 1;
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = tid; i < group * p.dv; i += 128) {
        const int head = kv_head * group + i / p.dv, c = i % p.dv;
        const size_t base = ((size_t)token * p.n_head + head) * p.splits;
        float mm = -INFINITY;
        for (int sp = 0; sp < live; ++sp) mm = fmaxf(mm, __ldcg(p.part_ml + (base + sp) * 2));
        float sum = 0.f, acc = 0.f;
        for (int sp = 0; sp < live; ++sp) {
            const float ms = __ldcg(p.part_ml + (base + sp) * 2);
            if (ms == -INFINITY) continue;
            const float f = exp2f(ms - mm);
            sum += f * __ldcg(p.part_ml + (base + sp) * 2 + 1);
            acc += f * __ldcg(p.part_o + (base + sp) * p.dv + c);
        }
        sum += sink_term(p, head, mm);
        acc = sum > 0.f ? acc / sum : 0.f;
        if (p.gate) acc *= logistic(__bfloat162float(p.gate[(size_t)token * p.gate_stride + (size_t)head * p.dv + c]));
        p.out[(size_t)token * p.n_head * p.dv + (size_t)head * p.dv + c] = __float2bfloat16_rn(acc);
    }
}

// out[token, head] = (sum over ranges of 2^(m_s - M) O_s) / (sum of 2^(m_s - M) l_s), times the gate.
// The ranges' maxima and sums come to shared memory in one trip, their weights are worked out there
// once, and every thread then sums its column over the ranges with independent loads.
constexpr int MERGE_MAX = 1024;   // most ranges (mg_attention_mma_split_keys keeps to it)

__global__ void attention_merge_kernel(const AttnParams p) {
    __shared__ float weight[MERGE_MAX];
    __shared__ float norm;
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)token * p.n_head + head) * p.splits;
    bf16* orow = p.out + (size_t)token * p.n_head * p.dv + (size_t)head * p.dv;
    const int position = p.positions[token];
    if (position < 0) {
        for (int c = threadIdx.x; c < p.dv; c += blockDim.x) orow[c] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo_row = first_visible(p, position);
    const int live = min(min(p.splits, MERGE_MAX), (position - (lo_row / KB) * KB) / p.split_keys + 1);   // ranges that hold keys
    for (int s = threadIdx.x; s < live; s += blockDim.x) weight[s] = p.part_ml[(base + s) * 2];
    __syncthreads();
    if (threadIdx.x < 32) {
        float mm = -INFINITY;
        for (int s = threadIdx.x; s < live; s += 32) mm = fmaxf(mm, weight[s]);
        mm = warp_max(mm);
        float sum = 0.f;
        for (int s = threadIdx.x; s < live; s += 32) {
            const float ms = weight[s];
            const float w = ms == -INFINITY ? 0.f : exp2f(ms - mm);
            weight[s] = w;
            sum += w * p.part_ml[(base + s) * 2 + 1];
        }
        sum = warp_sum(sum) + sink_term(p, head, mm);
        if (threadIdx.x == 0) norm = sum > 0.f ? 1.0f / sum : 0.f;
    }
    __syncthreads();
    const bf16* grow = p.gate ? p.gate + (size_t)token * p.gate_stride + (size_t)head * p.dv : nullptr;
    for (int c = threadIdx.x; c < p.dv; c += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < live; ++s) acc = fmaf(weight[s], p.part_o[(base + s) * p.dv + c], acc);
        acc *= norm;
        if (grow) acc *= logistic(__bfloat162float(grow[c]));
        orow[c] = __float2bfloat16_rn(acc);
    }
}


// ---- wide rows that hold their own values ------------------------------------------------------------
// Key rows of several hundred features whose first dv features are also the values (cached latents): too wide for
// query fragments and a whole row of results in one warp's registers.  A CTA of eight warps takes 32 rows, (token,
// head of the group) pairs in token order, and walks blocks of 64 keys (two buffers in turn).  The queries wait in
// shared memory.  Warp (rg, cg) takes rows 16 rg .. 16 rg + 15: it multiplies them with keys 16 cg .. 16 cg + 15 of the
// block, the four warps of a row group exchange their maxima through shared memory, each keeps the sum of its own
// keys' weights (the sums meet after the last block), the weights go to shared memory as bfloat16, and the warp
// then adds the block's 64 keys into columns CW cg .. CW cg + CW - 1 of its rows' results.  `single`: the rows are one
// token's heads and the CTA takes one range of its keys; results go to scratch as the merge kernel reads them.
constexpr int WIDE_ROWS = 32;

template <int CW>
__global__ void __launch_bounds__(256, 1)
attention_wide_kernel(const AttnParams p, const int single, const int dpad, const int row_tiles) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int stride = dpad + PAD;
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);                     // [32][stride]
    bf16* kbuf = qs + WIDE_ROWS * stride;                              // [2][KB][stride]
    bf16* ps = kbuf + 2 * KB * stride;                                 // [32][KB + PAD]
    float* mx = reinterpret_cast<float*>(ps + WIDE_ROWS * (KB + PAD)); // [4][32]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, rg = warp & 1, cg = warp >> 1;
    // columns d .. dpad of the key rows are never loaded: zeros, once
    if (p.d < dpad) {
        const int extra = dpad - p.d;
        for (int i = tid; i < 2 * KB * extra; i += 256) kbuf[(i / extra) * stride + p.d + i % extra] = __float2bfloat16_rn(0.f);
    }
    pdl_trigger();
    pdl_wait();
    const int kv_head = blockIdx.y, group = p.n_head / p.n_kv_head;
    int request, first_token, row_base, rows_total, j_first, j_last, lo_all;
    if (single) {
        const int token = blockIdx.x / row_tiles, split = blockIdx.z;
        int position = p.positions[token];
        if (position < 0) return;                                      // padding: the merge writes its zeros
        if (!MG_GUARDED(attention_mma, MG_GUARD_POSITION, position, (long long)p.max_pages * p.page_tokens)) position = 0;
        lo_all = first_visible(p, position);
        const int live = (position - (lo_all / KB) * KB) / p.split_keys + 1;
        if (split >= live) return;
        j_first = (lo_all / KB) * KB + split * p.split_keys;
        j_last = min(position, j_first + p.split_keys - 1);
        request = p.token_request[token];
        if (!MG_GUARDED(attention_mma, MG_GUARD_REQUEST, request, p.n_requests)) request = 0;
        first_token = token;
        row_base = (blockIdx.x % row_tiles) * WIDE_ROWS;
        rows_total = group;
    } else {
        int tile = (int)(gridDim.x - 1 - blockIdx.x);                   // the last tiles, which see the most keys, first
        for (request = 0; request < p.n_requests; ++request) {
            const int tiles = (p.req_q_len[request] * group + WIDE_ROWS - 1) / WIDE_ROWS;
            if (tile < tiles) break;
            tile -= tiles;
        }
        if (request >= p.n_requests) return;
        first_token = p.req_q_start[request];
        row_base = tile * WIDE_ROWS;
        rows_total = p.req_q_len[request] * group;
        const int last_row = min(rows_total, row_base + WIDE_ROWS) - 1;
        int hi = p.positions[first_token + last_row / group];
        if (hi < 0) return;                                            // padding
        if (!MG_GUARDED(attention_mma, MG_GUARD_POSITION, hi, (long long)p.max_pages * p.page_tokens)) hi = 0;
        lo_all = p.window > 0 ? first_visible(p, max(0, p.positions[first_token + row_base / group])) : 0;
        j_first = (lo_all / KB) * KB;
        j_last = hi;
    }
    const int* table = p.block_table + (size_t)request * p.max_pages;

    // the queries of the tile's rows; rows without a token and columns beyond d as zeros
    {
        const int chunks = dpad >> 3;
        for (int i = tid; i < WIDE_ROWS * chunks; i += 256) {
            const int r = i / chunks, c = (i - r * chunks) * 8, row = row_base + r;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row < rows_total && c < p.d) {
                const int t = single ? 0 : row / group, h = single ? row : row - t * group;
                v = *reinterpret_cast<const uint4*>(p.q + (size_t)(first_token + t) * p.q_stride + (size_t)(kv_head * group + h) * p.d + c);
            }
            *reinterpret_cast<uint4*>(qs + r * stride + c) = v;
        }
    }
    // this lane's two rows
    int pos[2], lo[2], token[2], head[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row_base + rg * 16 + (lane >> 2) + 8 * r;
        const bool live = row < rows_total;
        const int t = (single || !live) ? 0 : row / group;
        token[r] = first_token + t;
        head[r] = kv_head * group + (live ? row - t * group : 0);
        pos[r] = live ? p.positions[token[r]] : -1;
        lo[r] = pos[r] >= 0 ? first_visible(p, pos[r]) : 0;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[CW / 8][4];
#pragma unroll
    for (int n = 0; n < CW / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    const int page_shift = (p.page_tokens & (p.page_tokens - 1)) == 0 ? __ffs(p.page_tokens) - 1 : -1;
    const int chunks = p.d >> 3;
    // a warp copies eight of a block's keys, a row's 16-byte chunks across its lanes
    auto load_keys = [&](int j0, bf16* dst) {
        for (int key = warp * 8; key < warp * 8 + 8; ++key) {
            const int j = j0 + key;
            const bool real = j >= lo_all && j <= j_last;
            size_t row = 0;
            if (real) {
                const int index = page_shift >= 0 ? j >> page_shift : j / p.page_tokens;
                const int within = page_shift >= 0 ? j & (p.page_tokens - 1) : j - index * p.page_tokens;
                int page = table[index];
                if (!MG_GUARDED(attention_mma, MG_GUARD_PAGE, page, p.num_pages)) page = 0;
                row = ((size_t)page * p.n_kv_head + kv_head) * p.page_tokens + within;
            }
            for (int c = lane; c < chunks; c += 32) cp_async16(dst + key * stride + c * 8, p.k_pages + row * p.d + c * 8, real);
        }
    };
    load_keys(j_first, kbuf);
    cp_async_commit();
    int buf = 0;
    for (int j0 = j_first; j0 <= j_last; j0 += KB, buf ^= 1) {
        cp_async_wait<0>();
        __syncthreads();                                   // the block is here; everyone has left the one before
        if (j0 + KB <= j_last) {
            load_keys(j0 + KB, kbuf + (buf ^ 1) * KB * stride);
            cp_async_commit();
        }
        const bf16* kb = kbuf + buf * KB * stride;
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const bf16* a_ptr = qs + (rg * 16 + (lane & 15)) * stride + (lane >> 4) * 8;
        const bf16* b_ptr = kb + (cg * 16 + (lane >> 4) * 8 + (lane & 7)) * stride + ((lane >> 3) & 1) * 8;
#pragma unroll 4
        for (int kk = 0; kk < dpad; kk += 16) {
            uint32_t a[4], b[4];
            ldsm4(a, a_ptr + kk);
            ldsm4(b, b_ptr + kk);
            mma16816(s[0], a, b[0], b[1]);
            mma16816(s[1], a, b[2], b[3]);
        }
        float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + cg * 16 + n * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
                float sc = s[n][e] * p.scale_log2;
                if (p.cap_log2 > 0.f) sc = p.cap_log2 * tanhf(sc / p.cap_log2);
                const float v = (j <= pos[r] && j >= lo[r]) ? sc : -INFINITY;
                s[n][e] = v;
                bm[r] = fmaxf(bm[r], v);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 1));
            bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 2));
            if ((lane & 3) == 0) mx[cg * WIDE_ROWS + rg * 16 + (lane >> 2) + 8 * r] = bm[r];
        }
        __syncthreads();
        float corr[2], base[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = rg * 16 + (lane >> 2) + 8 * r;
            const float all = fmaxf(fmaxf(mx[row], mx[WIDE_ROWS + row]), fmaxf(mx[2 * WIDE_ROWS + row], mx[3 * WIDE_ROWS + row]));
            const float nm = fmaxf(m[r], all);
            corr[r] = (m[r] == -INFINITY) ? 0.f : exp2_approx(m[r] - nm);
            base[r] = (nm == -INFINITY) ? 0.f : nm;
            m[r] = nm;
        }
        float bs[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pr = exp2_approx(s[n][e] - base[e >> 1]);
                s[n][e] = pr;
                bs[e >> 1] += pr;
            }
#pragma unroll
            for (int r = 0; r < 2; ++r)
                *reinterpret_cast<uint32_t*>(ps + (rg * 16 + (lane >> 2) + 8 * r) * (KB + PAD) + cg * 16 + n * 8 + 2 * (lane & 3)) =
                    pack_bf16(s[n][2 * r], s[n][2 * r + 1]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            bs[r] += __shfl_xor_sync(0xffffffffu, bs[r], 1);
            bs[r] += __shfl_xor_sync(0xffffffffu, bs[r], 2);
            l[r] = l[r] * corr[r] + bs[r];
        }
#pragma unroll
        for (int n = 0; n < CW / 8; ++n) {
            o[n][0] *= corr[0];
            o[n][1] *= corr[0];
            o[n][2] *= corr[1];
            o[n][3] *= corr[1];
        }
        __syncthreads();                                   // all 64 keys' weights of the warp's rows are there
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
            uint32_t a[4];
            ldsm4(a, ps + (rg * 16 + (lane & 15)) * (KB + PAD) + kk * 16 + (lane >> 4) * 8);
            const bf16* v_ptr = kb + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * stride + cg * CW + (lane >> 4) * 8;
#pragma unroll
            for (int n = 0; n < CW / 8; n += 2) {
                uint32_t b[4];
                ldsm4_t(b, v_ptr + n * 8);
                mma16816(o[n], a, b[0], b[1]);
                mma16816(o[n + 1], a, b[2], b[3]);
            }
        }
    }
    // the four warps of a row group kept the sums of their own keys: they meet here
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r)
        if ((lane & 3) == 0) mx[cg * WIDE_ROWS + rg * 16 + (lane >> 2) + 8 * r] = l[r];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (pos[r] < 0) continue;
        const int row = rg * 16 + (lane >> 2) + 8 * r;
        float sum = mx[row] + mx[WIDE_ROWS + row] + mx[2 * WIDE_ROWS + row] + mx[3 * WIDE_ROWS + row];
        if (single) {
            const size_t slot = ((size_t)token[r] * p.n_head + head[r]) * p.splits + blockIdx.z;
            if (cg == 0 && (lane & 3) == 0) {
                p.part_ml[slot * 2] = m[r];
                p.part_ml[slot * 2 + 1] = sum;
            }
#pragma unroll
            for (int n = 0; n < CW / 8; ++n) {
                const int c = cg * CW + n * 8 + 2 * (lane & 3);
                if (c >= p.dv) continue;
                *reinterpret_cast<float2*>(p.part_o + slot * p.dv + c) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            }
            continue;
        }
        sum += sink_term(p, head[r], m[r]);
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        bf16* orow = p.out + (size_t)token[r] * p.n_head * p.dv + (size_t)head[r] * p.dv;
        const bf16* grow = p.gate ? p.gate + (size_t)token[r] * p.gate_stride + (size_t)head[r] * p.dv : nullptr;
#pragma unroll
        for (int n = 0; n < CW / 8; ++n) {
            const int c = cg * CW + n * 8 + 2 * (lane & 3);
            if (c >= p.dv) continue;
            float a = o[n][2 * r] * inv, b = o[n][2 * r + 1] * inv;
            if (grow) {
                const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(grow + c);
                a *= logistic(__bfloat162float(g.x));
                b *= logistic(__bfloat162float(g.y));
            }
            *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16(a, b);
        }
    }
}

template <int CW>
int launch_wide(const AttnParams& p, int single, int n_tiles, int dpad, size_t smem, cudaStream_t s) {
    const int group = p.n_head / p.n_kv_head, row_tiles = (group + WIDE_ROWS - 1) / WIDE_ROWS;
    cudaError_t e = cudaFuncSetAttribute(attention_wide_kernel<CW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
        const dim3 grid = single ? dim3(p.n_tokens * row_tiles, p.n_kv_head, p.splits) : dim3(n_tiles, p.n_kv_head);
        e = mg_launch(attention_wide_kernel<CW>, grid, dim3(256), smem, s, true, p, single, dpad, row_tiles);
    }
    if (e == cudaSuccess && single)
        e = mg_launch(attention_merge_kernel, dim3(p.n_tokens, p.n_head), dim3(128), 0, s, true, p);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (wide rows): %s", cudaGetErrorString(e));
    return MG_OK;
}

template <int DP, int DVP>
int launch(const AttnParams& p, int single_tokens, int n_tiles, cudaStream_t s) {
    size_t smem = (size_t)2 * KB * (DP + PAD + DVP + PAD) * sizeof(bf16);      // two buffers
    cudaError_t e;
    if (single_tokens) {
        const size_t meet = (size_t)(4 * 16 * 2 + 4 * 16 * DVP) * sizeof(float);
        if (meet > smem) smem = meet;
        e = cudaFuncSetAttribute(attention_split_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            e = mg_launch(attention_split_kernel<DP, DVP>, dim3(p.n_tokens, p.n_kv_head, p.splits), dim3(128), smem, s, true, p);
        if (e == cudaSuccess && p.counters == nullptr)
            e = mg_launch(attention_merge_kernel, dim3(p.n_tokens, p.n_head), dim3(p.dv >= 128 ? 128 : 64), 0, s, true, p);
    } else {
        e = cudaFuncSetAttribute(attention_tiles_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            e = mg_launch(attention_tiles_kernel<DP, DVP>, dim3(n_tiles, p.n_kv_head), dim3(128), smem, s, true, p);
    }
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "attention (mma): %s", cudaGetErrorString(e));
    return MG_OK;
}

}  // namespace

// Ranges of keys per token for contexts of up to max_context keys, and the keys per range.
MG_API int mg_attention_mma_split_keys(int max_context) {
    // short ranges: many CTAs with two blocks each (a CTA's blocks follow one another at a memory
    // round trip apiece); ranges beyond a token's own context leave at once, so the count only sizes
    // the grid and the scratch
    int keys = 128;
    while ((max_context + keys - 1) / keys > 1024) keys *= 2;
    return keys;
}

MG_API long long mg_attention_mma_scratch_floats(int n_tokens, int n_head, int dv, int splits) {
    return (long long)n_tokens * n_head * splits * (dv + 2);
}

// q: [n_tokens, q_stride] bfloat16 (heads of d features first); pages as in the general kernel;
// gate: rows of gate_stride elements or null; out: [n_tokens, n_head * dv] bfloat16.
// single_tokens = 1: every token is alone in its request's step (splits ranges of split_keys keys,
// scratch of mg_attention_mma_scratch_floats floats; counters: n_tokens * n_kv_head zeros that are left
// as zeros, or null to merge the ranges in a second kernel); 0: n_tiles tiles of tile_tokens tokens, found
// from req_q_start / req_q_len.  slopes: [n_head] 32-bit or null; key_block <= 0: no block mask; softcap <= 0: none;
// sinks: [n_head] 32-bit or null; v_stride: elements between value rows (0: dv).  Returns MG_ERR_UNSUPPORTED for sizes
// it does not take.
MG_API int mg_attention_mma(const void* q, int q_stride, const void* k_pages, const void* v_pages, const int* block_table,
                            const int* token_request, const int* positions, const int* req_q_start,
                            const int* req_q_len, const void* gate, int gate_stride, void* out, float* scratch,
                            int* counters, int n_tokens, int n_requests, int n_head, int n_kv_head, int d, int dv, int page_tokens,
                            int max_pages, int window, float scale, int num_pages, int single_tokens, int n_tiles,
                            int tile_tokens, int splits, int split_keys, const float* slopes, int key_block, float softcap,
                            const float* sinks, int v_stride, void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && n_head % n_kv_head == 0 && page_tokens > 0 && max_pages > 0,
               "attention: bad sizes");
    const int group = n_head / n_kv_head;
    if (v_stride <= 0) v_stride = dv;
    MG_REQUIRE(v_stride >= dv, "attention: value rows shorter than the values");
    const bool aligned = d % 8 == 0 && dv % 8 == 0 && v_stride % 8 == 0 && q_stride % 8 == 0 && (gate == nullptr || gate_stride % 2 == 0) &&
                         ((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pages % 16 == 0) && ((uintptr_t)v_pages % 16 == 0) &&
                         ((uintptr_t)out % 4 == 0) && ((uintptr_t)gate % 4 == 0);
    if (!aligned || d > 128 || dv > 128 || group > (single_tokens ? 16 : 64) || n_kv_head > 65535) return MG_ERR_UNSUPPORTED;
    AttnParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)v_pages;
    p.block_table = block_table; p.token_request = token_request; p.positions = positions;
    p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.gate = (const bf16*)gate; p.gate_stride = gate_stride;
    p.out = (bf16*)out; p.part_o = nullptr; p.part_ml = nullptr; p.counters = single_tokens ? counters : nullptr;
    p.n_tokens = n_tokens; p.n_requests = n_requests; p.n_head = n_head; p.n_kv_head = n_kv_head; p.d = d; p.dv = dv;
    p.page_tokens = page_tokens; p.max_pages = max_pages; p.window = window > 0 ? window : 0; p.num_pages = num_pages;
    p.tile_tokens = tile_tokens; p.splits = splits; p.split_keys = split_keys; p.scale_log2 = scale * LOG2E;
    p.slopes = slopes; p.block = key_block > 0 ? key_block : 0;
    p.cap_log2 = softcap > 0.f ? softcap * LOG2E : 0.f; p.sinks = sinks; p.v_stride = v_stride;
    if (single_tokens) {
        MG_REQUIRE(scratch != nullptr && splits > 0 && splits <= 65535 && split_keys > 0 && split_keys % KB == 0,
                   "attention: the ranges of keys want scratch and sizes that are multiples of %d", KB);
        p.part_o = scratch;
        p.part_ml = scratch + (size_t)n_tokens * n_head * splits * dv;
    } else {
        MG_REQUIRE(req_q_start && req_q_len && n_tiles > 0 && tile_tokens > 0 && tile_tokens * group <= 64,
                   "attention: tiles of up to 64 rows");
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int dp = d <= 64 ? 64 : d <= 96 ? 96 : 128, dvp = dv <= 64 ? 64 : 128;
    if (dp == 64 && dvp == 64) return launch<64, 64>(p, single_tokens, n_tiles, s);
    if (dp == 64) return launch<64, 128>(p, single_tokens, n_tiles, s);
    if (dp == 96 && dvp == 64) return launch<96, 64>(p, single_tokens, n_tiles, s);
    if (dp == 96) return launch<96, 128>(p, single_tokens, n_tiles, s);
    if (dvp == 64) return launch<128, 64>(p, single_tokens, n_tiles, s);
    return launch<128, 128>(p, single_tokens, n_tiles, s);
}

// Rows of 32 (token, head) pairs that the wide-row kernel takes for a prompt portion of `tokens` tokens.
MG_API int mg_attention_wide_tiles(int tokens, int group) { return (tokens * group + WIDE_ROWS - 1) / WIDE_ROWS; }

// Attention over key rows of d features whose first dv features are the values (one row per token and key/value
// head, k_pages [page, G, page_tokens, d]); the other arguments as mg_attention_mma.  single_tokens = 1: splits ranges
// of split_keys keys, scratch of mg_attention_mma_scratch_floats floats, merged by a second kernel; 0: n_tiles is the
// sum of mg_attention_wide_tiles over the requests.  Returns MG_ERR_UNSUPPORTED for sizes it does not take.
MG_API int mg_attention_wide(const void* q, int q_stride, const void* k_pages, const int* block_table, const int* token_request,
                             const int* positions, const int* req_q_start, const int* req_q_len, const void* gate,
                             int gate_stride, void* out, float* scratch, int n_tokens, int n_requests, int n_head, int n_kv_head,
                             int d, int dv, int page_tokens, int max_pages, int window, float scale, int num_pages,
                             int single_tokens, int n_tiles, int splits, int split_keys, float softcap, const float* sinks,
                             void* stream) {
    if (n_tokens == 0) return MG_OK;
    MG_REQUIRE(n_tokens > 0 && n_head > 0 && n_kv_head > 0 && n_head % n_kv_head == 0 && page_tokens > 0 && max_pages > 0 &&
               dv > 0 && dv <= d, "attention (wide rows): bad sizes");
    const bool aligned = d % 8 == 0 && dv % 8 == 0 && q_stride % 8 == 0 && (gate == nullptr || gate_stride % 2 == 0) &&
                         ((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pages % 16 == 0) && ((uintptr_t)out % 4 == 0) &&
                         ((uintptr_t)gate % 4 == 0);
    const int dpad = (d + 15) / 16 * 16;
    const size_t smem = ((size_t)(WIDE_ROWS + 2 * KB) * (dpad + PAD) + WIDE_ROWS * (KB + PAD)) * sizeof(bf16) + 4 * WIDE_ROWS * sizeof(float);
    if (!aligned || dv > 512 || smem > 227 * 1024 || n_kv_head > 65535) return MG_ERR_UNSUPPORTED;
    AttnParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.k_pages = (const bf16*)k_pages; p.v_pages = (const bf16*)k_pages;
    p.block_table = block_table; p.token_request = token_request; p.positions = positions;
    p.req_q_start = req_q_start; p.req_q_len = req_q_len; p.gate = (const bf16*)gate; p.gate_stride = gate_stride;
    p.out = (bf16*)out; p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr;
    p.n_tokens = n_tokens; p.n_requests = n_requests; p.n_head = n_head; p.n_kv_head = n_kv_head; p.d = d; p.dv = dv;
    p.page_tokens = page_tokens; p.max_pages = max_pages; p.window = window > 0 ? window : 0; p.num_pages = num_pages;
    p.tile_tokens = 0; p.splits = splits; p.split_keys = split_keys; p.scale_log2 = scale * LOG2E;
    p.slopes = nullptr; p.block = 0;
    p.cap_log2 = softcap > 0.f ? softcap * LOG2E : 0.f; p.sinks = sinks; p.v_stride = d;
    if (single_tokens) {
        MG_REQUIRE(scratch != nullptr && splits > 0 && splits <= 65535 && split_keys > 0 && split_keys % KB == 0,
                   "attention: the ranges of keys want scratch and sizes that are multiples of %d", KB);
        p.part_o = scratch;
        p.part_ml = scratch + (size_t)n_tokens * n_head * splits * dv;
    } else {
        MG_REQUIRE(req_q_start && req_q_len && n_tiles > 0, "attention (wide rows): no tiles");
    }
    cudaStream_t s = (cudaStream_t)stream;
    // the values' columns, padded, in four equal parts of whole pairs of 8-column tiles; padded columns lie inside
    // the padded key row (dv <= d) or, beyond it, in the row's padding and the next row: they are never stored
    if (dv <= 64 && dpad >= 64) return launch_wide<16>(p, single_tokens, n_tiles, dpad, smem, s);
    if (dv <= 128 && dpad >= 128) return launch_wide<32>(p, single_tokens, n_tiles, dpad, smem, s);
    if (dv <= 256 && dpad >= 256) return launch_wide<64>(p, single_tokens, n_tiles, dpad, smem, s);
    if (dpad >= 512) return launch_wide<128>(p, single_tokens, n_tiles, dpad, smem, s);
    return MG_ERR_UNSUPPORTED;
}
