// Attention whose heads talk to one another before the softmax, and whose values are its keys.
//
//   q = Wq h + bq,  k = Wk h + bk,  v = k as projected                      (H query heads on G key heads of D values)
//   q, k <- the first `rot` dimensions rotated by the position (pairs (i, i + rot/2)), then every head divided by its
//           root mean square over D (no weight)
//   s_h(i, j)  = cap * tanh(q_h(i) . k_g(j) * scale * temp_h / cap)           (cap 0: no bound)
//   s'_h(i, j) = sum_m talk[h][m] s_m(i, j)                                   (every head's score is a mix of all heads' scores)
//   i sees j <= i with i - j < window or j < keep_first (window 0: every j <= i);  p = softmax_j s'
//   out_h(i)   = gate_h(i) * sum_j p_h(i, j) v_g(j),   gate = sigmoid(Wg h), one number a value
//
// Because a score needs all heads' raw scores of the same (i, j), a block owns ALL heads of its rows: the raw scores of a
// tile of positions go through shared memory, and every head mixes its own from them.
//
//   prepare   from the fused projection [q | k | gate] (float): bias, rotation, unit norm, q in the activation type, k and the
//             unrotated, unnormed k (the values) into the cache's two planes at the row's position, gate = sigmoid (float)
//   rows      one block a row, one warp a head (two heads a warp past 32 heads): the true 32-bit path, any size, and the
//             checked twin of the tile kernel
//   tiles     bf16 on mma.sync tiles: a block (or a cluster of blocks) owns sixteen rows of one sequence and all heads; steps of
//             few rows a sequence share the positions out over several blocks, whose parts a second kernel merges
//
// Scores, the bound, the mix, the softmax's weights and all sums are float.  A row's sums run in an order that its position
// and the sizes alone fix, so a row gives the same bits in any batch and under any cut of its prompt.
#include <cooperative_groups.h>

#include "common.cuh"
#include "mma_tiles.cuh"

namespace cg = cooperative_groups;

#define TA_MAX_HEADS 64
#define TA_MAX_D 256

__device__ __forceinline__ float4 ta_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ta_load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

// ------------------------------------------------------------------------------------ prepare
// One block a row, one warp a head of q or of k at a time.  proj: [rows, P] float, q at 0 (H D), k at H D (G D), the gate's
// part at g_at (H D values); bias: [H D + G D] float or null.
template <class T>
__global__ void __launch_bounds__(256)
talk_prepare_kernel(const float* proj, int P, int g_at, const float* __restrict__ bias, const float* __restrict__ cos_sin, int table_positions,
                    const int* __restrict__ row_pos, const int* __restrict__ row_slot, const int* __restrict__ page_table, int max_pages,
                    int n_pages, T* __restrict__ q_out, T* k_cache, T* v_cache, float* __restrict__ gate, int H, int G, int D, int rot, float eps,
                    int write_cache) {
    __shared__ float xs[8][TA_MAX_D];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float* x = proj + (size_t)r * P;
    const int slot = row_slot[r], pos = row_pos[r];
    const int half = rot / 2;
    const bool turn = rot > 0 && cos_sin != nullptr && pos >= 0 && pos < table_positions;
    const float* cs = cos_sin + (size_t)(turn ? pos : 0) * half * 2;
    int page = -1;
    if (slot >= 0 && pos >= 0 && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    if (page >= n_pages) page = -1;
    const bool cache = write_cache && page >= 0;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) gate[(size_t)r * H * D + i] = 1.0f / (1.0f + expf(-x[g_at + i]));
    float* mine = xs[warp];
    for (int head = warp; head < H + G; head += warps) {
        const bool is_q = head < H;
        if (!is_q && !cache) continue;
        const float* xh = x + (size_t)head * D;          // the keys follow the queries in the projection
        const float* bh = bias ? bias + (size_t)head * D : nullptr;
        const size_t at = is_q ? 0 : (((size_t)page * G + (head - H)) * BC_PAGE + pos % BC_PAGE) * D;
        __syncwarp();
        for (int d = lane; d < D; d += 32) {
            const float v = xh[d] + (bh ? bh[d] : 0.0f);
            mine[d] = v;
            if (!is_q) v_cache[at + d] = from_f32<T>(v);  // the values are the keys as projected
        }
        __syncwarp();
        float ss = 0.0f;
        float keep[TA_MAX_D / 32];
#pragma unroll
        for (int j = 0; j < TA_MAX_D / 32; j++) {
            const int d = lane + 32 * j;
            float v = 0.0f;
            if (d < D) {
                v = mine[d];
                if (turn && d < rot) {
                    const int p = d < half ? d : d - half;
                    const float c = cs[2 * p], s = cs[2 * p + 1];
                    v = d < half ? v * c - mine[d + half] * s : v * c + mine[d - half] * s;
                }
                ss = fmaf(v, v, ss);
            }
            keep[j] = v;
        }
        ss = warp_sum(ss);
        const float f = 1.0f / sqrtf(ss / (float)D + eps);
        T* dst = is_q ? q_out + ((size_t)r * H + head) * D : k_cache + at;
#pragma unroll
        for (int j = 0; j < TA_MAX_D / 32; j++) {
            const int d = lane + 32 * j;
            if (d < D) dst[d] = from_f32<T>(keep[j] * f);
        }
    }
}

// --------------------------------------------------------------------------------------- rows
// One block a row; HPW heads a warp (warp w takes heads w, w + warps, ..); NJ value dimensions a lane (D <= 32 NJ).
// q: [rows, H, D]; k_cache, v_cache: [pages, G, BC_PAGE, D]; gate: [rows, H D] float; out: [rows, H D].
template <class T, int NJ, int HPW>
__global__ void __launch_bounds__(1024)
talk_rows_kernel(const T* q, const T* k_cache, const T* v_cache, const int* __restrict__ page_table, const int* __restrict__ row_pos,
                 const int* __restrict__ row_slot, const float* gate, const float* __restrict__ temp, const float* __restrict__ talk,
                 T* __restrict__ out, int H, int G, int D, int max_pages, int n_pages, int window, int keep_first, float scale, float cap) {
    extern __shared__ __align__(16) float ta_smem[];
    float* qs = ta_smem;                   // [H][D]
    float* raw = qs + (size_t)H * D;       // [H][32]: the tile's raw scores, bounded
    float* mix = raw + (size_t)H * 32;     // [H][H]
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(q); PDL_FRESH(k_cache); PDL_FRESH(v_cache); PDL_FRESH(gate);
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int slot = row_slot[r];
    if (slot < 0) {
        for (int i = threadIdx.x; i < H * D; i += blockDim.x) out[(size_t)r * H * D + i] = from_f32<T>(0.0f);
        return;
    }
    const int pos = row_pos[r];
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) qs[i] = to_f32(q[(size_t)r * H * D + i]);
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) mix[i] = talk[i];
    const int group = H / G;
    const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    const int first_end = min(keep_first, lo);       // positions [0, first_end) are seen although they lie before the window
    const int* pages = page_table + (size_t)slot * max_pages;
    float acc[HPW][NJ], m[HPW], l[HPW], factor[HPW];
#pragma unroll
    for (int a = 0; a < HPW; a++) {
        m[a] = -INFINITY, l[a] = 0.0f;
        const int h = warp + a * warps;
        factor[a] = h < H ? scale * temp[h] : 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; j++) acc[a][j] = 0.0f;
    }
    const bool four = D % 4 == 0;
    // Two stretches of positions: the kept first ones, then the window.
    for (int part = 0; part < 2; part++) {
        const int from = part == 0 ? 0 : lo, to = part == 0 ? first_end - 1 : pos;      // inclusive
        for (int t0 = from & ~31; t0 <= to; t0 += 32) {
            const int pi = t0 / BC_PAGE;
            int page = pi < max_pages ? pages[pi] : -1;
            if (page < 0 || page >= n_pages) page = -1;
            const int t = t0 + lane;
            const bool seen = page >= 0 && t >= from && t <= to;
            __syncthreads();                                    // the tile before has been read (and, the first time, qs and mix are whole)
#pragma unroll
            for (int a = 0; a < HPW; a++) {
                const int h = warp + a * warps;
                if (h >= H) continue;
                float s = 0.0f;
                if (seen) {
                    const T* kr = k_cache + (((size_t)page * G + h / group) * BC_PAGE + (t % BC_PAGE)) * D;
                    const float* qh = qs + (size_t)h * D;
                    if (four) {
                        for (int d = 0; d < D; d += 4) {
                            const float4 kv = ta_load4(kr + d);
                            const float4 qv = *reinterpret_cast<const float4*>(qh + d);
                            s = fmaf(kv.x, qv.x, s); s = fmaf(kv.y, qv.y, s); s = fmaf(kv.z, qv.z, s); s = fmaf(kv.w, qv.w, s);
                        }
                    } else {
                        for (int d = 0; d < D; d++) s = fmaf(to_f32(kr[d]), qh[d], s);
                    }
                    s *= factor[a];
                    if (cap > 0.0f) s = cap * tanhf(s / cap);
                }
                raw[h * 32 + lane] = s;
            }
            __syncthreads();
            const int count = page < 0 ? 0 : min(32, to + 1 - t0);
            const int begin = max(0, from - t0);
#pragma unroll
            for (int a = 0; a < HPW; a++) {
                const int h = warp + a * warps;
                if (h >= H) continue;
                float s = 0.0f;
                for (int mm = 0; mm < H; mm++) s = fmaf(mix[h * H + mm], raw[mm * 32 + lane], s);
                if (!seen) s = -INFINITY;
                const float mn = fmaxf(m[a], warp_max(s));
                const float corr = mn == -INFINITY ? 1.0f : expf(m[a] - mn);
                const float p = seen ? expf(s - mn) : 0.0f;
                l[a] = l[a] * corr + warp_sum(p);
#pragma unroll
                for (int j = 0; j < NJ; j++) acc[a][j] *= corr;
                const T* vt = v_cache + (((size_t)(page < 0 ? 0 : page) * G + h / group) * BC_PAGE + (t0 % BC_PAGE)) * D;
                for (int i = begin; i < count; i++) {
                    const float pi_ = __shfl_sync(0xffffffffu, p, i);
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int d = lane + 32 * j;
                        if (d < D) acc[a][j] = fmaf(pi_, to_f32(vt[(size_t)i * D + d]), acc[a][j]);
                    }
                }
                m[a] = mn;
            }
        }
    }
#pragma unroll
    for (int a = 0; a < HPW; a++) {
        const int h = warp + a * warps;
        if (h >= H) continue;
        const float inv = l[a] > 0.0f ? 1.0f / l[a] : 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int d = lane + 32 * j;
            if (d < D) out[((size_t)r * H + h) * D + d] = from_f32<T>(acc[a][j] * inv * gate[((size_t)r * H + h) * D + d]);
        }
    }
}

// -------------------------------------------------------------------------------------- tiles
// bf16 prompts.  A block owns sixteen rows of one sequence and all heads; warp w owns heads w, w + warps, .. (HPW of them).
// Positions come in tiles of 32 (half a page), keys and values of every kv head, through two stages of shared memory by
// cp.async.  A tile takes two passes with a barrier between them:
//   1. every warp multiplies its heads' queries with the tile's keys on m16n8k16 tiles, scales, bounds, and leaves the raw
//      scores (float) in shared memory;
//   2. every warp mixes its heads' scores out of all heads' raw ones (float), masks, takes the softmax's step (running maximum
//      and sum in registers), and multiplies the weights (bf16, out of its own registers) with the tile's values.
// The tiles a block walks: those of the kept first positions that lie before the window of its last row, then those from the
// window of its first row to its last row's own position.
// More than sixteen heads are shared out over a thread-block cluster of CL blocks (two up to 32 heads, four up to 64): a block
// owns H / CL heads and their kv heads (so a tile's keys and values are loaded once a cluster) and writes its heads' raw scores into
// every block's shared memory (distributed shared memory: one remote write an element, where reading the others' scores in place
// would be H / CL remote reads of each), so that every block mixes its heads' scores out of a copy of its own; the two barriers a
// tile are then the cluster's.
#define TT_KEYS 32
#define TT_ROWS 16
#define TT_RS 36            // floats a row of raw scores takes in shared memory.  A row keeps every thread's eight scores side by side
                            // ([quarter of the lane][n-block][2]), so that they move sixteen bytes at a time; four floats of
                            // padding a row let the eight threads of such an access meet no bank twice

__device__ __forceinline__ float tt_bound(float s, float cap, float two_over_cap) {
    // cap * tanh(s / cap) = cap * (1 - 2 / (e^(2 s / cap) + 1))
    const float e = __expf(s * two_over_cap);
    return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}

template <int D, int HPW, int CL>
__global__ void __launch_bounds__(512)
talk_tiles_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const int* __restrict__ page_table,
                  const int* __restrict__ seq_rows, const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const float* gate,
                  const float* __restrict__ temp, const float* __restrict__ talk, bf16* __restrict__ out, int H, int G, int max_pages, int n_pages,
                  int window, int keep_first, float scale, float cap, int stages, float* __restrict__ scratch, int splits) {
    constexpr int CHUNKS = D / 8, KD = D / 16, ND = D / 8;
    constexpr int HEAD_BYTES = TT_KEYS * D * 2;            // one kv head's 32 positions
    extern __shared__ __align__(128) uint8_t tt_smem[];
    // This block's heads and kv heads: all of them, or its share of the cluster's.
    const int rank = CL > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int HL = H / CL, GL = G / CL, h_first = rank * HL, g_first = rank * GL;
    const int plane = GL * HEAD_BYTES;                     // a tile's keys of this block's kv heads; their values follow
    float* raw = reinterpret_cast<float*>(tt_smem + (size_t)stages * 2 * plane);      // [H][16][TT_RS]: all heads' raw scores
    float* mix = raw + (size_t)H * TT_ROWS * TT_RS;        // [HL][H]: the rows of the mix that make this block's heads
    float* raw_of[CL];                                     // every block's copy of the raw scores, as this block writes them
#pragma unroll
    for (int c = 0; c < CL; c++) raw_of[c] = CL > 1 ? cg::this_cluster().map_shared_rank(raw, c) : raw;
    auto sync_heads = [&]() {                              // all heads' warps: the block's, or the cluster's
        if (CL > 1) cg::this_cluster().sync();
        else __syncthreads();
    };

    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(q); PDL_FRESH(k_cache); PDL_FRESH(v_cache); PDL_FRESH(gate);
    const int sq = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int gq = lane >> 2, tq = lane & 3, j4 = lane >> 3, r8 = lane & 7;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    const int n_tiles_q = (n_new + TT_ROWS - 1) / TT_ROWS;
    const int q_tile = n_tiles_q - 1 - (int)blockIdx.x / CL;    // the last rows see the most: they go first
    if (slot < 0 || q_tile < 0) return;                    // (the same for every block of a cluster)
    const int start = seq_start[sq];
    const int tok0 = q_tile * TT_ROWS, tok_end = min(n_new, tok0 + TT_ROWS);
    const int* pages = page_table + (size_t)slot * max_pages;
    const int group = H / G;
    const int last_pos = start + n_new - 1;                // the last position the sequence holds after this step

    for (int i = threadIdx.x; i < HL * H; i += blockDim.x) mix[i] = talk[(size_t)h_first * H + i];
    auto first_seen = [&](int p) { return window > 0 && p + 1 > window ? p + 1 - window : 0; };
    int pos[2], lo[2];
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int tok = tok0 + gq + 8 * i;
        live[i] = tok < n_new;
        pos[i] = start + tok;
        lo[i] = first_seen(pos[i]);
    }
    // The block's tiles of positions: [0, kept) and [win_begin, win_end], as one stretch where they meet.
    const int p_first = start + tok0, p_last = start + tok_end - 1;
    int kept = (min(keep_first, first_seen(p_last)) + TT_KEYS - 1) / TT_KEYS;
    const int win_begin = first_seen(p_first) / TT_KEYS, win_end = p_last / TT_KEYS;
    if (kept >= win_begin) kept = win_begin;
    const int all_tiles = kept + (win_end - win_begin + 1);
    // With several splits (few rows a sequence: single rows above all) block z walks its share of the tiles and leaves its
    // maxima, sums and products in scratch memory for the merge.
    const int per_split = (all_tiles + splits - 1) / splits;
    const int tile_first = (int)blockIdx.z * per_split;
    const int n_tiles = max(0, min(all_tiles, tile_first + per_split) - tile_first);
    auto tile_at = [&](int k) { k += tile_first; return k < kept ? k : win_begin + (k - kept); };
    auto page_of = [&](int tile) {
        const int pi = tile / 2;
        const int page = pi < max_pages ? pages[pi] : -1;
        return page >= 0 && page < n_pages ? page : -1;
    };
    auto load_tile = [&](int tile, int stage) {
        const int page = page_of(tile);
        if (page < 0) return;
        const uint32_t kb = ad_smem(tt_smem + (size_t)stage * 2 * plane), vb = kb + plane;
        const int per_head = TT_KEYS * CHUNKS;
        for (int i = threadIdx.x; i < GL * per_head; i += blockDim.x) {
            const int g = i / per_head, rest = i - g * per_head, row = rest / CHUNKS, c = rest - row * CHUNKS;
            const size_t src = (((size_t)page * G + g_first + g) * BC_PAGE + (tile & 1) * TT_KEYS + row) * D + c * 8;
            cp_async16(kb + g * HEAD_BYTES + tile_offset<D>(row, c), k_cache + src);
            cp_async16(vb + g * HEAD_BYTES + tile_offset<D>(row, c), v_cache + src);
        }
    };

    // This warp's heads: queries as fragments, what each score is multiplied by, and the sums that run over the tiles.
    uint32_t qf[HPW][KD][4];
    float o[HPW][ND][4], m[HPW][2], l[HPW][2], factor[HPW];
#pragma unroll
    for (int a = 0; a < HPW; a++) {
        const int hl = warp + a * warps, h = h_first + hl;      // the head's number in this block, and in the model
        factor[a] = hl < HL ? scale * temp[h] : 0.0f;
#pragma unroll
        for (int kd = 0; kd < KD; kd++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const bf16* qr = q + ((size_t)(row0 + tok0 + gq + 8 * i) * H + (hl < HL ? h : 0)) * D + kd * 16 + 2 * tq;
                const bool ok = live[i] && hl < HL;
                qf[a][kd][i] = ok ? *reinterpret_cast<const uint32_t*>(qr) : 0u;
                qf[a][kd][i + 2] = ok ? *reinterpret_cast<const uint32_t*>(qr + 8) : 0u;
            }
#pragma unroll
        for (int nd = 0; nd < ND; nd++) o[a][nd][0] = o[a][nd][1] = o[a][nd][2] = o[a][nd][3] = 0.0f;
        m[a][0] = m[a][1] = -INFINITY;
        l[a][0] = l[a][1] = 0.0f;
    }
    const float two_over_cap = cap > 0.0f ? 2.0f / cap : 0.0f;
    const float LOG2E = 1.4426950408889634f;

    if (n_tiles > 0) load_tile(tile_at(0), 0);
    cp_async_commit();
    for (int it = 0; it < n_tiles; it++) {
        const int stage = stages > 1 ? (it & 1) : 0;
        if (stages == 1 && it > 0) {
            __syncthreads();                               // everybody has left the tile before
            load_tile(tile_at(it), 0);
            cp_async_commit();
        }
        cp_async_wait<0>();
        sync_heads();                                      // the tile has come, and nobody reads the raw scores of the tile before any more (so they may be overwritten, from any block)
        if (stages > 1 && it + 1 < n_tiles) load_tile(tile_at(it + 1), stage ^ 1);
        cp_async_commit();
        const int tile = tile_at(it);
        if (page_of(tile) < 0) continue;                   // a tile without a page is neither fetched nor multiplied
        const uint32_t kb = ad_smem(tt_smem + (size_t)stage * 2 * plane), vb = kb + plane;
        if (tile == last_pos / TT_KEYS && last_pos % TT_KEYS != TT_KEYS - 1) {
            // What lies past the sequence's last position belongs to nobody (a sequence that held the page before may have left
            // not-a-numbers there, and 0 x NaN is NaN in the product with the values): those value rows are cleared in the copy.
            const int first = last_pos % TT_KEYS + 1;
            for (int i = threadIdx.x; i < GL * (TT_KEYS - first) * CHUNKS; i += blockDim.x) {
                const int g = i / ((TT_KEYS - first) * CHUNKS), rest = i - g * (TT_KEYS - first) * CHUNKS;
                *reinterpret_cast<uint4*>(tt_smem + (size_t)stage * 2 * plane + plane + g * HEAD_BYTES + tile_offset<D>(first + rest / CHUNKS, rest % CHUNKS)) =
                    make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();
        }
        // 1. raw scores of this warp's heads
#pragma unroll
        for (int a = 0; a < HPW; a++) {
            const int hl = warp + a * warps, h = h_first + hl;
            if (hl >= HL) continue;
            const uint32_t kh = kb + (h / group - g_first) * HEAD_BYTES;
            float s[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
            for (int kd = 0; kd < KD; kd++)
#pragma unroll
                for (int np = 0; np < 2; np++) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(kh + tile_offset<D>(np * 16 + (j4 >> 1) * 8 + r8, kd * 2 + (j4 & 1)), b0, b1, b2, b3);
                    mma_16816(s[2 * np], qf[a][kd], b0, b1);
                    mma_16816(s[2 * np + 1], qf[a][kd], b2, b3);
                }
#pragma unroll
            for (int nb = 0; nb < 4; nb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s[nb][e] *= factor[a];
                    if (cap > 0.0f) s[nb][e] = tt_bound(s[nb][e], cap, two_over_cap);
                }
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const float4 v = make_float4(s[2 * half][2 * i], s[2 * half][2 * i + 1], s[2 * half + 1][2 * i], s[2 * half + 1][2 * i + 1]);
#pragma unroll
                    for (int c = 0; c < CL; c++)
                        *reinterpret_cast<float4*>(raw_of[c] + (size_t)h * TT_ROWS * TT_RS + (gq + 8 * i) * TT_RS + tq * 8 + half * 4) = v;
                }
        }
        sync_heads();
        // 2. this warp's heads: the mix of all heads' raw scores, the softmax's step, the product with the values
#pragma unroll
        for (int a = 0; a < HPW; a++) {
            const int hl = warp + a * warps, h = h_first + hl;
            if (hl >= HL) continue;
            float s[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
            const float* mh = mix + (size_t)hl * H;
#pragma unroll 4
            for (int mm = 0; mm < H; mm++) {
                const float f = mh[mm];
                const float* rm = raw + (size_t)mm * TT_ROWS * TT_RS;
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const float4 v = *reinterpret_cast<const float4*>(rm + (gq + 8 * i) * TT_RS + tq * 8 + half * 4);
                        s[2 * half][2 * i] = fmaf(f, v.x, s[2 * half][2 * i]);
                        s[2 * half][2 * i + 1] = fmaf(f, v.y, s[2 * half][2 * i + 1]);
                        s[2 * half + 1][2 * i] = fmaf(f, v.z, s[2 * half + 1][2 * i]);
                        s[2 * half + 1][2 * i + 1] = fmaf(f, v.w, s[2 * half + 1][2 * i + 1]);
                    }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 4; nb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int i = e >> 1;
                    const int t = tile * TT_KEYS + nb * 8 + 2 * tq + (e & 1);
                    const bool seen = live[i] && t <= pos[i] && (t >= lo[i] || t < keep_first);
                    s[nb][e] = seen ? s[nb][e] * LOG2E : -INFINITY;
                    tmax[i] = fmaxf(tmax[i], s[nb][e]);
                }
            float corr[2], base[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
                tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
                const float mn = fmaxf(m[a][i], tmax[i]);
                corr[i] = mn == -INFINITY ? 1.0f : fast_exp2(m[a][i] - mn);
                base[i] = mn == -INFINITY ? 0.0f : mn;
                m[a][i] = mn;
            }
            float psum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int nb = 0; nb < 4; nb++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s[nb][e] = fast_exp2(s[nb][e] - base[e >> 1]);
                    psum[e >> 1] += s[nb][e];
                }
            l[a][0] = l[a][0] * corr[0] + psum[0];
            l[a][1] = l[a][1] * corr[1] + psum[1];
#pragma unroll
            for (int nd = 0; nd < ND; nd++) {
                o[a][nd][0] *= corr[0]; o[a][nd][1] *= corr[0]; o[a][nd][2] *= corr[1]; o[a][nd][3] *= corr[1];
            }
            const uint32_t vh = vb + (h / group - g_first) * HEAD_BYTES;
#pragma unroll
            for (int kk = 0; kk < 2; kk++) {
                const uint32_t pf[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int nd = 0; nd < ND; nd += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vh + tile_offset<D>(kk * 16 + (j4 & 1) * 8 + r8, nd + (j4 >> 1)), b0, b1, b2, b3);
                    mma_16816(o[a][nd], pf, b0, b1);
                    mma_16816(o[a][nd + 1], pf, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    if (CL > 1) cg::this_cluster().sync();                 // no block leaves while another may still write raw scores into its memory
#pragma unroll
    for (int a = 0; a < HPW; a++) {
        const int hl = warp + a * warps, h = h_first + hl;
        if (hl >= HL) continue;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float sum = l[a][i];
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (!live[i]) continue;
            if (splits > 1) {
                float* part = scratch + (((size_t)(row0 + tok0 + gq + 8 * i) * H + h) * splits + blockIdx.z) * (D + 2);
                if (tq == 0) part[0] = m[a][i], part[1] = sum;
#pragma unroll
                for (int nd = 0; nd < ND; nd++) *reinterpret_cast<float2*>(part + 2 + nd * 8 + 2 * tq) = make_float2(o[a][nd][2 * i], o[a][nd][2 * i + 1]);
                continue;
            }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            const size_t at = ((size_t)(row0 + tok0 + gq + 8 * i) * H + h) * D + 2 * tq;
#pragma unroll
            for (int nd = 0; nd < ND; nd++) {
                const float2 gv = *reinterpret_cast<const float2*>(gate + at + nd * 8);
                *reinterpret_cast<uint32_t*>(out + at + nd * 8) = pack_bf16(o[a][nd][2 * i] * inv * gv.x, o[a][nd][2 * i + 1] * inv * gv.y);
            }
        }
    }
}

// One block a (row, head): the splits' maxima (in powers of two), sums and products in the order of the splits, then the gate.
__global__ void __launch_bounds__(128)
talk_merge_kernel(const float* scratch, const int* __restrict__ row_slot, const float* gate, bf16* __restrict__ out, int H, int D, int splits) {
    __shared__ float wz[64];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(scratch); PDL_FRESH(gate);
    const int r = blockIdx.x, h = blockIdx.y;
    const size_t at = ((size_t)r * H + h) * D;
    if (row_slot[r] < 0) {
        for (int d = threadIdx.x; d < D; d += blockDim.x) out[at + d] = __float2bfloat16_rn(0.0f);
        return;
    }
    const float* part = scratch + ((size_t)r * H + h) * splits * (D + 2);
    float top = -INFINITY;
    for (int z = 0; z < splits; z++) top = fmaxf(top, part[(size_t)z * (D + 2)]);
    if (threadIdx.x < splits) {
        const float mz = part[(size_t)threadIdx.x * (D + 2)];
        wz[threadIdx.x] = mz == -INFINITY ? 0.0f : fast_exp2(mz - top);
    }
    __syncthreads();
    float total = 0.0f;
    for (int z = 0; z < splits; z++) total += wz[z] * part[(size_t)z * (D + 2) + 1];
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int z = 0; z < splits; z++) {
            const float w = wz[z];
            if (w > 0.0f) acc = fmaf(w, part[(size_t)z * (D + 2) + 2 + d], acc);      // a split that saw nothing may hold anything
        }
        out[at + d] = __float2bfloat16_rn(acc * inv * gate[at + d]);
    }
}

extern "C" long long bc_talk_tiles_scratch_floats(int rows, int H, int D, int splits) {
    return splits <= 1 ? 0 : (long long)rows * H * splits * (D + 2);
}

// Shared memory of one block that owns H / CL heads and G / CL kv heads.
static size_t tt_smem_bytes(int H, int G, int D, int stages, int CL) {
    return (size_t)stages * 2 * (G / CL) * TT_KEYS * D * 2 + ((size_t)H * TT_ROWS * TT_RS + (size_t)(H / CL) * H) * sizeof(float);
}
// How the heads are shared out: (blocks a cluster, heads a warp), or (0, 0) where the tiles do not take these sizes.  One block of
// up to sixteen warps, a head each; more heads as a cluster of two or four such blocks, where heads and kv heads divide evenly;
// else two heads a warp in one block, whose accumulators then hold 2 D value columns a thread (D up to 64).
static void tt_shape(int H, int G, int D, int* CL, int* HPW) {
    *CL = *HPW = 0;
    if (H <= 0 || G <= 0 || H % G || D % 16 || D < 16 || D > 128) return;
    if (H <= 16) { *CL = 1, *HPW = 1; return; }
    for (int c = 2; c <= 4; c *= 2)
        if (H <= 16 * c && H % c == 0 && G % c == 0) { *CL = c, *HPW = 1; return; }
    if (H <= 32 && D <= 64) *CL = 1, *HPW = 2;
}

extern "C" int bc_talk_tiles_accepts(int H, int G, int D) {
    int CL, HPW;
    tt_shape(H, G, D, &CL, &HPW);
    return CL > 0 && tt_smem_bytes(H, G, D, 1, CL) <= 216 * 1024;
}

template <int D, int HPW, int CL>
static int tiles_go(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* seq_rows, const int* seq_slot,
                    const int* seq_start, const float* gate, const float* temp, const float* talk, void* out, int seqs, int max_new, int H, int G,
                    int max_pages, int n_pages, int window, int keep_first, float scale, float cap, float* scratch, int splits, const int* row_slot,
                    int rows, cudaStream_t s) {
    const int stages = tt_smem_bytes(H, G, D, 2, CL) <= 216 * 1024 ? 2 : 1;
    const size_t smem = tt_smem_bytes(H, G, D, stages, CL);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(talk_tiles_kernel<D, HPW, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            bc_set_error("talk_tiles: cannot set shared memory to %zu: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured = smem;
    }
    const int warps = (H / CL + HPW - 1) / HPW;
    const dim3 grid(((max_new + TT_ROWS - 1) / TT_ROWS) * CL, seqs, splits);
    cudaError_t e;
    if (CL > 1)
        e = bc_launch_clustered(talk_tiles_kernel<D, HPW, CL>, grid, dim3(32 * warps), smem, s, dim3(CL, 1, 1), (const bf16*)q, (const bf16*)k_cache,
                                (const bf16*)v_cache, page_table, seq_rows, seq_slot, seq_start, gate, temp, talk, (bf16*)out, H, G, max_pages, n_pages,
                                window, keep_first, scale, cap, stages, scratch, splits);
    else
        e = bc_launch(talk_tiles_kernel<D, HPW, CL>, grid, dim3(32 * warps), smem, s, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                      page_table, seq_rows, seq_slot, seq_start, gate, temp, talk, (bf16*)out, H, G, max_pages, n_pages, window, keep_first, scale, cap,
                      stages, scratch, splits);
    if (e != cudaSuccess) {
        bc_set_error("talk_tiles: %s", cudaGetErrorString(e));
        return (int)e;
    }
    if (splits > 1) bc_launch(talk_merge_kernel, dim3(rows, H), dim3(128), 0, s, (const float*)scratch, row_slot, gate, (bf16*)out, H, D, splits);
    BC_LAUNCH_STATUS();
}

// q: [rows, H D] bf16; k_cache, v_cache: [pages, G, BC_PAGE, D] bf16; gate: [rows, H D] float; temp: [H]; talk: [H, H]; out: [rows, H D] bf16.
// Sequence s brings rows seq_rows[s] .. seq_rows[s + 1] and held seq_start[s] positions before.  splits > 1 (few rows a sequence): the
// tiles of positions a block would walk are shared out over that many blocks, which leave their parts in scratch (floats as
// bc_talk_tiles_scratch_floats says) for a second kernel; then row_slot [rows] tells which of the `rows` rows of q belong to no sequence.
extern "C" int bc_talk_tiles_bf16(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* seq_rows, const int* seq_slot,
                                  const int* seq_start, const float* gate, const float* temp, const float* talk, void* out, int seqs, int max_new, int H,
                                  int G, int D, int max_pages, int n_pages, int window, int keep_first, float scale, float cap, float* scratch, int splits,
                                  const int* row_slot, int rows, cudaStream_t s) {
    BC_CHECK_ARG(splits >= 1 && splits <= 64 && (splits == 1 || (scratch && row_slot && rows >= 0)), "talk_tiles: %d splits (1 to 64) or their scratch", splits);
    BC_CHECK_ARG(bc_talk_tiles_accepts(H, G, D), "talk_tiles: %d heads on %d of %d are not taken (heads of multiples of 16 up to 128; up to 16 heads, "
                 "or up to 64 where a cluster of two or four blocks shares heads and kv heads out evenly)", H, G, D);
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && max_new >= 0 && window >= 0 && keep_first >= 0 && cap >= 0.0f && temp && talk && gate,
                 "talk_tiles: bad sizes seqs=%d max_new=%d window=%d kept=%d", seqs, max_new, window, keep_first);
    if (seqs == 0 || max_new == 0) return BC_OK;
    int CL, HPW;
    tt_shape(H, G, D, &CL, &HPW);
#define TT_GO(DD, HH, CC) return tiles_go<DD, HH, CC>(q, k_cache, v_cache, page_table, seq_rows, seq_slot, seq_start, gate, temp, talk, out, seqs, max_new, H, \
                                                      G, max_pages, n_pages, window, keep_first, scale, cap, scratch, splits, row_slot, rows, s)
#define TT_D(DD)                         \
    case DD:                             \
        if (CL == 2) TT_GO(DD, 1, 2);    \
        if (CL == 4) TT_GO(DD, 1, 4);    \
        if (HPW == 1) TT_GO(DD, 1, 1);   \
        break;
    if (HPW == 2) {
        switch (D) {
            case 16: TT_GO(16, 2, 1);
            case 32: TT_GO(32, 2, 1);
            case 48: TT_GO(48, 2, 1);
            case 64: TT_GO(64, 2, 1);
        }
    }
    switch (D) { TT_D(16) TT_D(32) TT_D(48) TT_D(64) TT_D(80) TT_D(96) TT_D(112) TT_D(128) }
#undef TT_D
#undef TT_GO
    bc_set_error("talk_tiles: heads of %d are not taken", D);
    return BC_ERR_ARG;
}

// ---------------------------------------------------------------------------------- launchers
template <class T>
static int prepare(const float* proj, int rows, int P, int g_at, const float* bias, const float* cos_sin, int table_positions, const int* row_pos,
                   const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out, void* k_cache, void* v_cache, float* gate,
                   int H, int G, int D, int rot, float eps, int write_cache, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && D > 0 && D <= TA_MAX_D && eps > 0.0f, "talk_prepare: bad sizes rows=%d H=%d G=%d D=%d (at most %d)", rows, H,
                 G, D, TA_MAX_D);
    BC_CHECK_ARG(rot >= 0 && rot % 2 == 0 && rot <= D && (rot == 0 || cos_sin), "talk_prepare: %d rotated dimensions of a head of %d", rot, D);
    BC_CHECK_ARG((H + G) * D <= P && g_at >= 0 && g_at + H * D <= P, "talk_prepare: the parts do not fit a row of %d", P);
    if (rows == 0) return BC_OK;
    const int heads = H + G;
    const int threads = heads >= 8 ? 256 : heads >= 4 ? 128 : 64;      // by the row's heads alone
    bc_launch(talk_prepare_kernel<T>, dim3(rows), dim3(threads), 0, s, proj, P, g_at, bias, cos_sin, table_positions, row_pos, row_slot, page_table,
              max_pages, n_pages, (T*)q_out, (T*)k_cache, (T*)v_cache, gate, H, G, D, rot, eps, write_cache);
    BC_LAUNCH_STATUS();
}
// proj: [rows, P] float; bias: [(H + G) D] float or null; cos_sin: [table_positions, rot / 2, 2] float; q_out: [rows, H D];
// k_cache, v_cache: [pages, G, BC_PAGE, D]; gate: [rows, H D] float.  Rows whose slot is negative write no cache.
extern "C" int bc_talk_prepare_f32(const float* proj, int rows, int P, int g_at, const float* bias, const float* cos_sin, int table_positions,
                                   const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out,
                                   void* k_cache, void* v_cache, float* gate, int H, int G, int D, int rot, float eps, int write_cache, cudaStream_t s) {
    return prepare<float>(proj, rows, P, g_at, bias, cos_sin, table_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache, v_cache,
                          gate, H, G, D, rot, eps, write_cache, s);
}
extern "C" int bc_talk_prepare_bf16(const float* proj, int rows, int P, int g_at, const float* bias, const float* cos_sin, int table_positions,
                                    const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out,
                                    void* k_cache, void* v_cache, float* gate, int H, int G, int D, int rot, float eps, int write_cache, cudaStream_t s) {
    return prepare<bf16>(proj, rows, P, g_at, bias, cos_sin, table_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache, v_cache,
                         gate, H, G, D, rot, eps, write_cache, s);
}

template <class T, int NJ, int HPW>
static int rows_go(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos, const int* row_slot,
                   const float* gate, const float* temp, const float* talk, void* out, int rows, int H, int G, int D, int max_pages, int n_pages,
                   int window, int keep_first, float scale, float cap, cudaStream_t s) {
    const int warps = (H + HPW - 1) / HPW;
    const size_t smem = ((size_t)H * D + (size_t)H * 32 + (size_t)H * H) * sizeof(float);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(talk_rows_kernel<T, NJ, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            bc_set_error("talk_rows: cannot set shared memory to %zu: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured = smem;
    }
    bc_launch(talk_rows_kernel<T, NJ, HPW>, dim3(rows), dim3(32 * warps), smem, s, (const T*)q, (const T*)k_cache, (const T*)v_cache, page_table, row_pos,
              row_slot, gate, temp, talk, (T*)out, H, G, D, max_pages, n_pages, window, keep_first, scale, cap);
    BC_LAUNCH_STATUS();
}

template <class T>
static int rows_launch(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos, const int* row_slot,
                       const float* gate, const float* temp, const float* talk, void* out, int rows, int H, int G, int D, int max_pages, int n_pages,
                       int window, int keep_first, float scale, float cap, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= TA_MAX_HEADS && G > 0 && H % G == 0 && D > 0 && D <= TA_MAX_D,
                 "talk_rows: bad sizes rows=%d H=%d (at most %d) G=%d D=%d (at most %d)", rows, H, TA_MAX_HEADS, G, D, TA_MAX_D);
    BC_CHECK_ARG(window >= 0 && keep_first >= 0 && cap >= 0.0f && temp && talk && gate, "talk_rows: bad window %d, kept positions %d or bound %g", window,
                 keep_first, (double)cap);
    if (rows == 0) return BC_OK;
#define TA_GO(NJ, HPW) return rows_go<T, NJ, HPW>(q, k_cache, v_cache, page_table, row_pos, row_slot, gate, temp, talk, out, rows, H, G, D, max_pages, \
                                                  n_pages, window, keep_first, scale, cap, s)
    if (H <= 32) {
        if (D <= 64) TA_GO(2, 1);
        if (D <= 128) TA_GO(4, 1);
        TA_GO(8, 1);
    }
    if (D <= 64) TA_GO(2, 2);
    if (D <= 128) TA_GO(4, 2);
    TA_GO(8, 2);
#undef TA_GO
}
// q: [rows, H D]; k_cache, v_cache: [pages, G, BC_PAGE, D]; gate: [rows, H D] float; temp: [H] float; talk: [H, H] float;
// out: [rows, H D].  window 0: every earlier position; cap 0: scores are not bounded.
extern "C" int bc_talk_rows_f32(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos, const int* row_slot,
                                const float* gate, const float* temp, const float* talk, void* out, int rows, int H, int G, int D, int max_pages,
                                int n_pages, int window, int keep_first, float scale, float cap, cudaStream_t s) {
    return rows_launch<float>(q, k_cache, v_cache, page_table, row_pos, row_slot, gate, temp, talk, out, rows, H, G, D, max_pages, n_pages, window,
                              keep_first, scale, cap, s);
}
extern "C" int bc_talk_rows_bf16(const void* q, const void* k_cache, const void* v_cache, const int* page_table, const int* row_pos, const int* row_slot,
                                 const float* gate, const float* temp, const float* talk, void* out, int rows, int H, int G, int D, int max_pages,
                                 int n_pages, int window, int keep_first, float scale, float cap, cudaStream_t s) {
    return rows_launch<bf16>(q, k_cache, v_cache, page_table, row_pos, row_slot, gate, temp, talk, out, rows, H, G, D, max_pages, n_pages, window,
                             keep_first, scale, cap, s);
}
