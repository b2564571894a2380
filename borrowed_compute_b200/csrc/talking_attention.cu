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
//   rows      one block a row, one warp a head (two heads a warp past 32 heads): the true 32-bit path, the path of single
//             rows (a row sees at most window + keep_first positions), and the checked twin of the tile kernel
//   tiles     bf16 prompts on mma.sync tiles: a block owns sixteen rows of one sequence and all heads
//
// Scores, the bound, the mix, the softmax's weights and all sums are float.  A row's sums run in an order that its position
// and the sizes alone fix, so a row gives the same bits in any batch and under any cut of its prompt.
#include "common.cuh"
#include "mma_tiles.cuh"

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
