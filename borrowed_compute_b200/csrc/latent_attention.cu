// Latent attention: every head's keys and values are products of one cached vector a position.
//
// A position keeps c (R values, the normed down projection of the layer's input) and, if the mixer rotates, one
// rotated key part r (ROT values) that all heads share.  Head n's key is [Wuk_n c | r] and its value Wuv_n c, so
//     score_n(i, j) = (q_n . Wuk_n c_j + qr_n . r_j) * scale = ((Wuk_n^T q_n) . c_j + qr_n . r_j) * scale
//     out_n(i)      = Wuv_n (sum_j p_n(i, j) c_j)
// and attention runs over the cache as it is: every head reads the same R + ROT values a position (one "kv head"),
// with the absorbed query a_n = Wuk_n^T q_n on the left and c as the value; Wuv comes after the sum over positions.
//
//   prepare   from the fused down projection [q part | c and r part | gate part] (float): cq = N(q part) in the
//             activation type, c = N(c part) and the rotated r into the cache at the row's position, gate = sigmoid
//   query     a[r][n] = [Wuk_n^T q_n | rot(qr_n)] from the float up projection of cq
//   rows      attention, one warp a (row, head): the true 32-bit path and the checked twin of the tile kernel
//   values    out[r][n] = gate[r][n] * Wuv_n ctx[r][n]
//
// Cache layout of one layer: c [page][BC_PAGE][R], r [page][BC_PAGE][ROT]; page_table[slot][i] names the page of
// positions 64 i .. 64 i + 63.  Rows whose slot is negative are padding: they write nothing into the cache.
// Every sum of a row runs in an order that the sizes alone fix, so a row gives the same bits in any batch and cut.
#include "common.cuh"

#define LAT_MAX_R 512
#define LAT_MAX_ROT 128

__device__ __forceinline__ float4 lat_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 lat_load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

__device__ __forceinline__ float2 lat_load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 lat_load2(const bf16* p) {
    const unsigned raw = *reinterpret_cast<const unsigned*>(p);
    return make_float2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
}

// ------------------------------------------------------------------------------------ prepare
// One block a row.  proj: [rows, P] float; the q part starts at 0 and is QR wide, the c part at kv_at (R wide, then
// ROT values of r; kv_at < 0: the mixer reads another layer's cache and has no such part), the gate part at g_at (H wide).
template <class T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* proj, int P, int QR, int kv_at, int R, int ROT, int g_at, int H, const float* __restrict__ q_w,
                      const float* __restrict__ kv_w, const float* __restrict__ cos_sin, int table_positions, const int* __restrict__ row_pos,
                      const int* __restrict__ row_slot, const int* __restrict__ page_table, int max_pages, int n_pages, T* c_pages, T* r_pages,
                      T* __restrict__ cq, float* __restrict__ gate, float eps, int write) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int r = blockIdx.x;
    const float* x = proj + (size_t)r * P;
    float s = 0.0f;
#pragma unroll 4
    for (int i = threadIdx.x; i < QR; i += blockDim.x) s = fmaf(x[i], x[i], s);
    s = block_sum(s, scratch);
    const float qs = 1.0f / sqrtf(s / (float)QR + eps);
#pragma unroll 4
    for (int i = threadIdx.x; i < QR; i += blockDim.x) cq[(size_t)r * QR + i] = from_f32<T>(x[i] * qs * q_w[i]);
    for (int i = threadIdx.x; i < H; i += blockDim.x) gate[(size_t)r * H + i] = 1.0f / (1.0f + expf(-x[g_at + i]));
    if (kv_at < 0 || !write) return;
    const int slot = row_slot[r], pos = row_pos[r];
    if (slot < 0 || pos < 0) return;
    const int pi = pos / BC_PAGE;
    const int page = pi < max_pages ? page_table[(size_t)slot * max_pages + pi] : -1;
    const float* z = x + kv_at;
    float t = 0.0f;
#pragma unroll 4
    for (int i = threadIdx.x; i < R; i += blockDim.x) t = fmaf(z[i], z[i], t);
    t = block_sum(t, scratch);
    if (page < 0 || page >= n_pages) return;
    const float cs = 1.0f / sqrtf(t / (float)R + eps);
    const size_t at = (size_t)page * BC_PAGE + pos % BC_PAGE;
#pragma unroll 4
    for (int i = threadIdx.x; i < R; i += blockDim.x) c_pages[at * R + i] = from_f32<T>(z[i] * cs * kv_w[i]);
    if (ROT > 0 && pos < table_positions) {
        const int half = ROT / 2;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float2 f = *reinterpret_cast<const float2*>(cos_sin + ((size_t)pos * half + i) * 2);
            const float u = z[R + i], v = z[R + half + i];
            r_pages[at * ROT + i] = from_f32<T>(u * f.x - v * f.y);
            r_pages[at * ROT + half + i] = from_f32<T>(v * f.x + u * f.y);
        }
    }
}

// -------------------------------------------------------------------------------------- query
// Block (x, y, z): rows LQ_ROWS x .. of head y, columns LQ_COLS z .. of the latent.  q: [rows, H, D + ROT] float; w_uk: [H * D, R];
// a: [rows, H, R + ROT].  A lane owns two neighbouring columns and a warp every fourth query dimension, so that few rows
// still spread over heads * R / LQ_COLS blocks and a thread's loads of the matrix are independent; the warps' parts are
// added through shared memory.  The block of the first columns also rotates the rotated part.
#define LQ_ROWS 8
#define LQ_COLS 64
template <class T>
__global__ void __launch_bounds__(128)
latent_query_kernel(const float* q, const T* __restrict__ w_uk, const float* __restrict__ cos_sin, int table_positions, const int* __restrict__ row_pos,
                    T* __restrict__ a, int rows, int H, int D, int ROT, int R) {
    extern __shared__ float lq_q[];      // [LQ_ROWS][D], then the warps' parts [4][LQ_ROWS][LQ_COLS]
    float* part = lq_q + LQ_ROWS * D;
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(q);
    const int r0 = blockIdx.x * LQ_ROWS, h = blockIdx.y, n0 = blockIdx.z * LQ_COLS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int QW = D + ROT, AW = R + ROT;
    for (int i = threadIdx.x; i < LQ_ROWS * D; i += blockDim.x) {
        const int rr = r0 + i / D;
        lq_q[i] = rr < rows ? q[((size_t)rr * H + h) * QW + i % D] : 0.0f;
    }
    __syncthreads();
    const T* w = w_uk + (size_t)h * D * R;
    const int n = n0 + 2 * lane;
    const bool pair = R % 2 == 0;        // then every row of the matrix starts at an even element, and n is even
    float acc[LQ_ROWS][2];
#pragma unroll
    for (int i = 0; i < LQ_ROWS; i++) acc[i][0] = acc[i][1] = 0.0f;
    if (n < R) {
#pragma unroll 4
        for (int d = warp; d < D; d += 4) {
            float w0, w1 = 0.0f;
            if (pair) {
                const float2 two = lat_load2(w + (size_t)d * R + n);
                w0 = two.x, w1 = two.y;
            } else {
                w0 = to_f32(w[(size_t)d * R + n]);
                if (n + 1 < R) w1 = to_f32(w[(size_t)d * R + n + 1]);
            }
#pragma unroll
            for (int i = 0; i < LQ_ROWS; i++) {
                const float qv = lq_q[i * D + d];
                acc[i][0] = fmaf(qv, w0, acc[i][0]);
                acc[i][1] = fmaf(qv, w1, acc[i][1]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < LQ_ROWS; i++) {
        part[(warp * LQ_ROWS + i) * LQ_COLS + 2 * lane] = acc[i][0];
        part[(warp * LQ_ROWS + i) * LQ_COLS + 2 * lane + 1] = acc[i][1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < LQ_ROWS * LQ_COLS; i += blockDim.x) {
        const int rr = r0 + i / LQ_COLS, c = n0 + i % LQ_COLS;
        if (rr < rows && c < R)
            a[((size_t)rr * H + h) * AW + c] = from_f32<T>(part[i] + part[LQ_ROWS * LQ_COLS + i] + part[2 * LQ_ROWS * LQ_COLS + i] + part[3 * LQ_ROWS * LQ_COLS + i]);
    }
    if (blockIdx.z != 0) return;
    const int half = ROT / 2;
    for (int i = threadIdx.x; i < LQ_ROWS * half; i += blockDim.x) {
        const int rr = r0 + i / half, p = i % half;
        if (rr >= rows) continue;
        const int pos = row_pos[rr];
        const float* qr = q + ((size_t)rr * H + h) * QW + D;
        float2 f = make_float2(1.0f, 0.0f);
        if (pos >= 0 && pos < table_positions) f = *reinterpret_cast<const float2*>(cos_sin + ((size_t)pos * half + p) * 2);
        const float u = qr[p], v = qr[half + p];
        T* o = a + ((size_t)rr * H + h) * AW + R;
        o[p] = from_f32<T>(u * f.x - v * f.y);
        o[half + p] = from_f32<T>(v * f.x + u * f.y);
    }
}

// --------------------------------------------------------------------------------------- rows
template <class T> __device__ __forceinline__ float lat_dot(const T* k, const float* q, int n) {
    float s = 0.0f;
    if (n % 4 == 0) {
        for (int d = 0; d < n; d += 4) {
            const float4 kv = lat_load4(k + d);
            const float4 qv = *reinterpret_cast<const float4*>(q + d);
            s = fmaf(kv.x, qv.x, s); s = fmaf(kv.y, qv.y, s); s = fmaf(kv.z, qv.z, s); s = fmaf(kv.w, qv.w, s);
        }
    } else {
        for (int d = 0; d < n; d++) s = fmaf(to_f32(k[d]), q[d], s);
    }
    return s;
}

#define LR_WARPS 4
// One warp a (row, head): scores lanes-over-positions, values lanes-over-dimensions, a running maximum and sum.
// a: [rows, H, R + ROT]; out: [rows, H, R]; sink: [H] float or null (one more term e^sink of every row's sum).  NJ = the value dimensions a lane keeps (R <= 32 NJ).
template <class T, int NJ>
__global__ void __launch_bounds__(LR_WARPS * 32)
latent_rows_kernel(const T* a, const T* c_pages, const T* r_pages, const int* __restrict__ page_table, const int* __restrict__ row_pos,
                   const int* __restrict__ row_slot, T* __restrict__ out, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale,
                   const float* __restrict__ sink) {
    __shared__ __align__(16) float qs[LR_WARPS][LAT_MAX_R + LAT_MAX_ROT];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(a); PDL_FRESH(c_pages); PDL_FRESH(r_pages);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x, h = blockIdx.y * LR_WARPS + warp;
    if (h >= H) return;
    T* o = out + ((size_t)r * H + h) * R;
    const int slot = row_slot[r];
    if (slot < 0) {
        for (int d = lane; d < R; d += 32) o[d] = from_f32<T>(0.0f);
        return;
    }
    const int pos = row_pos[r];
    const T* ah = a + ((size_t)r * H + h) * (R + ROT);
    // The rotated part starts on a 16-byte border of its own in shared memory.
    float* qc = qs[warp];
    float* qr = qs[warp] + LAT_MAX_R;
    for (int d = lane; d < R; d += 32) qc[d] = to_f32(ah[d]);
    for (int d = lane; d < ROT; d += 32) qr[d] = to_f32(ah[R + d]);
    __syncwarp();
    const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    const int* pages = page_table + (size_t)slot * max_pages;
    float acc[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) acc[j] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    for (int t0 = lo & ~31; t0 <= pos; t0 += 32) {
        const int pi = t0 / BC_PAGE;
        int page = pi < max_pages ? pages[pi] : -1;
        if (page < 0 || page >= n_pages) page = -1;
        const size_t at = (size_t)(page < 0 ? 0 : page) * BC_PAGE + (t0 % BC_PAGE);
        const int t = t0 + lane;
        const bool seen = page >= 0 && t >= lo && t <= pos;
        float s = -INFINITY;
        if (seen) {
            s = lat_dot<T>(c_pages + (at + lane) * R, qc, R);
            if (ROT > 0) s += lat_dot<T>(r_pages + (at + lane) * ROT, qr, ROT);
            s *= scale;
        }
        const float mn = fmaxf(m, warp_max(s));
        const float corr = mn == -INFINITY ? 1.0f : expf(m - mn);
        const float p = seen ? expf(s - mn) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int j = 0; j < NJ; j++) acc[j] *= corr;
        const int count = page < 0 ? 0 : min(32, pos + 1 - t0);
        const T* vt = c_pages + at * R;
        for (int i = max(0, lo - t0); i < count; i++) {
            const float pi_ = __shfl_sync(0xffffffffu, p, i);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int d = lane + 32 * j;
                if (d < R) acc[j] = fmaf(pi_, to_f32(vt[(size_t)i * R + d]), acc[j]);
            }
        }
        m = mn;
    }
    // A sink is one more term of the row's sum, e^(the head's number - m), with no key and no value.
    if (sink != nullptr && m != -INFINITY) l += expf(sink[h] - m);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int d = lane + 32 * j;
        if (d < R) o[d] = from_f32<T>(acc[j] * inv);
    }
}

// ------------------------------------------------------------------------------------- values
// Block (x, y, z): rows LV_ROWS x .. of head y, value channels LV_CH z .. ; a warp takes every fourth of those channels and adds
// over R with its lanes (four values a load where R allows it), so that few rows spread over heads * DV / LV_CH blocks.
// ctx: [rows, H, R]; w_uv: [H * DV, R]; gate: [rows, H] float; out: [rows, H * DV].
#define LV_ROWS 8
#define LV_CH 16
template <class T>
__global__ void __launch_bounds__(128)
latent_values_kernel(const T* ctx, const T* __restrict__ w_uv, const float* gate, T* __restrict__ out, int rows, int H, int R, int DV) {
    extern __shared__ __align__(16) float lv_c[];      // [LV_ROWS][R]
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(ctx); PDL_FRESH(gate);
    const int r0 = blockIdx.x * LV_ROWS, h = blockIdx.y, v0 = blockIdx.z * LV_CH;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool four = R % 4 == 0;
    if (four) {
        // Four values a load, and the loads of a thread independent of one another: with few rows this fill is the kernel's
        // longest chain of memory round trips otherwise.
        const int R4 = R / 4;
#pragma unroll 4
        for (int i = threadIdx.x; i < LV_ROWS * R4; i += 128) {
            const int row = i / R4, c = i - row * R4;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (r0 + row < rows) v = lat_load4(ctx + ((size_t)(r0 + row) * H + h) * R + 4 * c);
            *reinterpret_cast<float4*>(lv_c + row * R + 4 * c) = v;
        }
    } else {
        for (int i = threadIdx.x; i < LV_ROWS * R; i += blockDim.x) {
            const int rr = r0 + i / R;
            lv_c[i] = rr < rows ? to_f32(ctx[((size_t)rr * H + h) * R + i % R]) : 0.0f;
        }
    }
    __syncthreads();
    // A warp's channels are v0 + warp + 4 j; they run side by side so that their loads of the matrix overlap.
    constexpr int CW = LV_CH / 4;
    const int v_end = min(v0 + LV_CH, DV);
    float acc[CW][LV_ROWS];
#pragma unroll
    for (int j = 0; j < CW; j++)
#pragma unroll
        for (int i = 0; i < LV_ROWS; i++) acc[j][i] = 0.0f;
    const T* w = w_uv + (size_t)h * DV * R;
    if (four) {
        for (int n = 4 * lane; n < R; n += 128) {
            float4 wv[CW];
#pragma unroll
            for (int j = 0; j < CW; j++) {
                const int v = v0 + warp + 4 * j;
                wv[j] = v < v_end ? lat_load4(w + (size_t)v * R + n) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int i = 0; i < LV_ROWS; i++) {
                const float4 c = *reinterpret_cast<const float4*>(lv_c + i * R + n);
#pragma unroll
                for (int j = 0; j < CW; j++) acc[j][i] = fmaf(c.x, wv[j].x, fmaf(c.y, wv[j].y, fmaf(c.z, wv[j].z, fmaf(c.w, wv[j].w, acc[j][i]))));
            }
        }
    } else {
        for (int n = lane; n < R; n += 32) {
#pragma unroll
            for (int j = 0; j < CW; j++) {
                const int v = v0 + warp + 4 * j;
                const float wv = v < v_end ? to_f32(w[(size_t)v * R + n]) : 0.0f;
#pragma unroll
                for (int i = 0; i < LV_ROWS; i++) acc[j][i] = fmaf(lv_c[i * R + n], wv, acc[j][i]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CW; j++) {
        const int v = v0 + warp + 4 * j;
#pragma unroll
        for (int i = 0; i < LV_ROWS; i++) {
            const float sum = warp_sum(acc[j][i]);
            if (lane == 0 && v < v_end && r0 + i < rows) out[(size_t)(r0 + i) * H * DV + (size_t)h * DV + v] = from_f32<T>(sum * gate[(size_t)(r0 + i) * H + h]);
        }
    }
}

// ---------------------------------------------------------------------------------- launchers
template <class T>
static int prepare(const float* proj, int rows, int P, int QR, int kv_at, int R, int ROT, int g_at, int H, const float* q_w, const float* kv_w,
                   const float* cos_sin, int table_positions, const int* row_pos, const int* row_slot, const int* page_table, int max_pages,
                   int n_pages, void* c_pages, void* r_pages, void* cq, float* gate, float eps, int write, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && P > 0 && QR > 0 && R > 0 && ROT >= 0 && ROT % 2 == 0 && H > 0 && eps > 0.0f,
                 "latent_prepare: bad sizes rows=%d P=%d q=%d c=%d rot=%d heads=%d", rows, P, QR, R, ROT, H);
    BC_CHECK_ARG(QR <= P && g_at >= 0 && g_at + H <= P && (kv_at < 0 || kv_at + R + ROT <= P), "latent_prepare: the parts do not fit a row of %d", P);
    BC_CHECK_ARG(kv_at < 0 || !write || (c_pages && page_table && (ROT == 0 || (r_pages && cos_sin))), "latent_prepare: a cache to write is missing");
    if (rows == 0) return BC_OK;
    bc_launch(latent_prepare_kernel<T>, dim3(rows), dim3(128), 0, s, proj, P, QR, kv_at, R, ROT, g_at, H, q_w, kv_w, cos_sin, table_positions, row_pos,
              row_slot, page_table, max_pages, n_pages, (T*)c_pages, (T*)r_pages, (T*)cq, gate, eps, write);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_latent_prepare_f32(const float* proj, int rows, int P, int QR, int kv_at, int R, int ROT, int g_at, int H, const float* q_w,
                                     const float* kv_w, const float* cos_sin, int table_positions, const int* row_pos, const int* row_slot,
                                     const int* page_table, int max_pages, int n_pages, void* c_pages, void* r_pages, void* cq, float* gate, float eps,
                                     int write, cudaStream_t s) {
    return prepare<float>(proj, rows, P, QR, kv_at, R, ROT, g_at, H, q_w, kv_w, cos_sin, table_positions, row_pos, row_slot, page_table, max_pages,
                          n_pages, c_pages, r_pages, cq, gate, eps, write, s);
}
extern "C" int bc_latent_prepare_bf16(const float* proj, int rows, int P, int QR, int kv_at, int R, int ROT, int g_at, int H, const float* q_w,
                                      const float* kv_w, const float* cos_sin, int table_positions, const int* row_pos, const int* row_slot,
                                      const int* page_table, int max_pages, int n_pages, void* c_pages, void* r_pages, void* cq, float* gate, float eps,
                                      int write, cudaStream_t s) {
    return prepare<bf16>(proj, rows, P, QR, kv_at, R, ROT, g_at, H, q_w, kv_w, cos_sin, table_positions, row_pos, row_slot, page_table, max_pages,
                         n_pages, c_pages, r_pages, cq, gate, eps, write, s);
}

template <class T>
static int query(const float* q, const void* w_uk, const float* cos_sin, int table_positions, const int* row_pos, void* a, int rows, int H, int D, int ROT,
                 int R, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && R > 0 && ROT >= 0 && ROT % 2 == 0, "latent_query: bad sizes rows=%d H=%d D=%d R=%d rot=%d", rows,
                 H, D, R, ROT);
    BC_CHECK_ARG(ROT == 0 || cos_sin, "latent_query: a rotation needs its table");
    const size_t shared = ((size_t)LQ_ROWS * D + 4 * LQ_ROWS * LQ_COLS) * sizeof(float);
    BC_CHECK_ARG(shared <= 48 * 1024 && (R + LQ_COLS - 1) / LQ_COLS <= 65535, "latent_query: heads of %d or a latent of %d are wider than this kernel takes", D, R);
    if (rows == 0) return BC_OK;
    bc_launch(latent_query_kernel<T>, dim3((rows + LQ_ROWS - 1) / LQ_ROWS, H, (R + LQ_COLS - 1) / LQ_COLS), dim3(128), shared, s, q, (const T*)w_uk, cos_sin,
              table_positions, row_pos, (T*)a, rows, H, D, ROT, R);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_latent_query_f32(const float* q, const void* w_uk, const float* cos_sin, int table_positions, const int* row_pos, void* a, int rows,
                                   int H, int D, int ROT, int R, cudaStream_t s) {
    return query<float>(q, w_uk, cos_sin, table_positions, row_pos, a, rows, H, D, ROT, R, s);
}
extern "C" int bc_latent_query_bf16(const float* q, const void* w_uk, const float* cos_sin, int table_positions, const int* row_pos, void* a, int rows,
                                    int H, int D, int ROT, int R, cudaStream_t s) {
    return query<bf16>(q, w_uk, cos_sin, table_positions, row_pos, a, rows, H, D, ROT, R, s);
}

template <class T>
static int rows_launch(const void* a, const void* c_pages, const void* r_pages, const int* page_table, const int* row_pos, const int* row_slot, void* out,
                       int rows, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale, const float* sink, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && R > 0 && R <= LAT_MAX_R && ROT >= 0 && ROT <= LAT_MAX_ROT && window >= 0,
                 "latent_rows: bad sizes rows=%d H=%d R=%d (at most %d) rot=%d (at most %d)", rows, H, R, LAT_MAX_R, ROT, LAT_MAX_ROT);
    BC_CHECK_ARG((H + LR_WARPS - 1) / LR_WARPS <= 65535 && (ROT == 0 || r_pages), "latent_rows: too many heads (%d) or no rotated keys", H);
    if (rows == 0) return BC_OK;
    dim3 grid(rows, (H + LR_WARPS - 1) / LR_WARPS);
#define LR_GO(NJ)                                                                                                                                   \
    bc_launch(latent_rows_kernel<T, NJ>, grid, dim3(LR_WARPS * 32), 0, s, (const T*)a, (const T*)c_pages, (const T*)r_pages, page_table, row_pos, \
              row_slot, (T*)out, H, R, ROT, max_pages, n_pages, window, scale, sink)
    if (R <= 128) LR_GO(4);
    else if (R <= 256) LR_GO(8);
    else LR_GO(16);
#undef LR_GO
    BC_LAUNCH_STATUS();
}
extern "C" int bc_latent_rows_f32(const void* a, const void* c_pages, const void* r_pages, const int* page_table, const int* row_pos, const int* row_slot,
                                  void* out, int rows, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale, const float* sink,
                                  cudaStream_t s) {
    return rows_launch<float>(a, c_pages, r_pages, page_table, row_pos, row_slot, out, rows, H, R, ROT, max_pages, n_pages, window, scale, sink, s);
}
extern "C" int bc_latent_rows_bf16(const void* a, const void* c_pages, const void* r_pages, const int* page_table, const int* row_pos, const int* row_slot,
                                   void* out, int rows, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale, const float* sink,
                                   cudaStream_t s) {
    return rows_launch<bf16>(a, c_pages, r_pages, page_table, row_pos, row_slot, out, rows, H, R, ROT, max_pages, n_pages, window, scale, sink, s);
}

template <class T>
static int values(const void* ctx, const void* w_uv, const float* gate, void* out, int rows, int H, int R, int DV, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && R > 0 && DV > 0, "latent_values: bad sizes rows=%d H=%d R=%d DV=%d", rows, H, R, DV);
    BC_CHECK_ARG((size_t)LV_ROWS * R * sizeof(float) <= 48 * 1024, "latent_values: a latent of %d is wider than this kernel takes", R);
    if (rows == 0) return BC_OK;
    bc_launch(latent_values_kernel<T>, dim3((rows + LV_ROWS - 1) / LV_ROWS, H, (DV + LV_CH - 1) / LV_CH), dim3(128), (size_t)LV_ROWS * R * sizeof(float), s, (const T*)ctx,
              (const T*)w_uv, gate, (T*)out, rows, H, R, DV);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_latent_values_f32(const void* ctx, const void* w_uv, const float* gate, void* out, int rows, int H, int R, int DV, cudaStream_t s) {
    return values<float>(ctx, w_uv, gate, out, rows, H, R, DV, s);
}
extern "C" int bc_latent_values_bf16(const void* ctx, const void* w_uv, const float* gate, void* out, int rows, int H, int R, int DV, cudaStream_t s) {
    return values<bf16>(ctx, w_uv, gate, out, rows, H, R, DV, s);
}
