// Latent attention for prompts, bf16: with many rows a sequence it is cheaper to expand the cached latents into every
// head's keys and values once (one product over the positions the step sees) than to move the key products to every
// query, so a prompt step gathers what it sees from the cache, multiplies it by [Wuk; Wuv], lays the result out as pages
// of per-head keys [Wuk_n c | r] and values Wuv_n c, and runs the library's prompt attention kernels over those.
//
//   heads    q (float, [rows, H, D + ROT]) -> bf16 [rows, H, KP]: D plain values, ROT rotated by the row's position, zeros
//   gather   the cache's rows of every scratch page (a slot's 64 positions from a multiple of 64) -> [S, R] and [S, ROT];
//            rows past the sequence's last position, and pages the cache no longer holds, are zeros
//   spread   kv [S, H D + H DV] and the gathered r -> keys [S / 64, H, 64, KP] and values [S / 64, H, 64, VP], zero padded
//   gate     out [rows, H, VP] times sigmoid gate [rows, H] -> [rows, H DV]
//
// KP and VP are widths the attention kernels take; the zeros change no score and the padded value columns are dropped.
#include "common.cuh"

// One block a row.
__global__ void __launch_bounds__(128)
latent_heads_kernel(const float* q, const float* __restrict__ cos_sin, int table_positions, const int* __restrict__ row_pos, bf16* __restrict__ out, int H,
                    int D, int ROT, int KP) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(q);
    const int r = blockIdx.x, QW = D + ROT, half = ROT / 2;
    const int pos = row_pos[r];
    const bool turn = pos >= 0 && pos < table_positions;
    for (int i = threadIdx.x; i < H * KP; i += blockDim.x) {
        const int h = i / KP, d = i - h * KP;
        const float* qh = q + ((size_t)r * H + h) * QW;
        float v = 0.0f;
        if (d < D) v = qh[d];
        else if (d < QW) {
            const int p = d - D, pair = p < half ? p : p - half;
            float2 f = make_float2(1.0f, 0.0f);
            if (turn) f = *reinterpret_cast<const float2*>(cos_sin + ((size_t)pos * half + pair) * 2);
            const float u = qh[D + pair], w = qh[D + half + pair];
            v = p < half ? u * f.x - w * f.y : w * f.x + u * f.y;
        }
        out[(size_t)r * H * KP + i] = __float2bfloat16_rn(v);
    }
}

// One block a scratch page.  pg_slot, pg_pos, pg_last: the slot whose positions pg_pos .. pg_pos + 63 the page takes, and
// the last position that slot holds.
__global__ void __launch_bounds__(128)
latent_gather_kernel(const bf16* c_pages, const bf16* r_pages, const int* __restrict__ page_table, const int* __restrict__ pg_slot,
                     const int* __restrict__ pg_pos, const int* __restrict__ pg_last, bf16* __restrict__ ctx_c, bf16* __restrict__ ctx_r, int R, int ROT,
                     int max_pages, int n_pages) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(c_pages); PDL_FRESH(r_pages);
    const int p = blockIdx.x, slot = pg_slot[p], pos0 = pg_pos[p], last = pg_last[p];
    const int pi = pos0 / BC_PAGE;
    int page = slot >= 0 && pi < max_pages ? page_table[(size_t)slot * max_pages + pi] : -1;
    if (page >= n_pages) page = -1;
    const int live = page < 0 ? 0 : min(BC_PAGE, last - pos0 + 1);
    const int CR = R / 8, CT = ROT / 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < BC_PAGE * CR; i += blockDim.x) {
        const int row = i / CR, c = i - row * CR;
        uint4 v = zero;
        if (row < live) v = *reinterpret_cast<const uint4*>(c_pages + ((size_t)page * BC_PAGE + row) * R + c * 8);
        *reinterpret_cast<uint4*>(ctx_c + ((size_t)p * BC_PAGE + row) * R + c * 8) = v;
    }
    for (int i = threadIdx.x; i < BC_PAGE * CT; i += blockDim.x) {
        const int row = i / CT, c = i - row * CT;
        uint4 v = zero;
        if (row < live) v = *reinterpret_cast<const uint4*>(r_pages + ((size_t)page * BC_PAGE + row) * ROT + c * 8);
        *reinterpret_cast<uint4*>(ctx_r + ((size_t)p * BC_PAGE + row) * ROT + c * 8) = v;
    }
}

// Block (x, y): gathered row x, heads 8 y .. ; a thread writes one value at a time, neighbours in a row of the output.
#define LS_HEADS 8
__global__ void __launch_bounds__(256)
latent_spread_kernel(const bf16* kv, const bf16* ctx_r, bf16* __restrict__ keys, bf16* __restrict__ values, int H, int D, int DV, int ROT, int KP, int VP) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(kv); PDL_FRESH(ctx_r);
    const size_t t = blockIdx.x;
    const int h0 = blockIdx.y * LS_HEADS, hn = min(LS_HEADS, H - h0);
    const size_t page = t / BC_PAGE, row = t % BC_PAGE;
    const bf16* src = kv + t * ((size_t)H * (D + DV));
    const bf16* rot = ctx_r + t * ROT;
    const bf16 zero = __float2bfloat16_rn(0.0f);
    if (D % 8 == 0 && DV % 8 == 0 && ROT % 8 == 0 && KP % 8 == 0 && VP % 8 == 0) {
        // Eight values (16 bytes) a thread: every part starts at a multiple of eight values, in the source and in the pages.
        const uint4 none = make_uint4(0u, 0u, 0u, 0u);
        const int KC = KP / 8, VC = VP / 8;
        for (int i = threadIdx.x; i < hn * KC; i += blockDim.x) {
            const int h = h0 + i / KC, d = 8 * (i % KC);
            uint4 v = none;
            if (d < D) v = *reinterpret_cast<const uint4*>(src + (size_t)h * D + d);
            else if (d < D + ROT) v = *reinterpret_cast<const uint4*>(rot + (d - D));
            *reinterpret_cast<uint4*>(keys + ((page * H + h) * BC_PAGE + row) * KP + d) = v;
        }
        for (int i = threadIdx.x; i < hn * VC; i += blockDim.x) {
            const int h = h0 + i / VC, d = 8 * (i % VC);
            uint4 v = none;
            if (d < DV) v = *reinterpret_cast<const uint4*>(src + (size_t)H * D + (size_t)h * DV + d);
            *reinterpret_cast<uint4*>(values + ((page * H + h) * BC_PAGE + row) * VP + d) = v;
        }
        return;
    }
    for (int i = threadIdx.x; i < hn * KP; i += blockDim.x) {
        const int h = h0 + i / KP, d = i % KP;
        keys[((page * H + h) * BC_PAGE + row) * KP + d] = d < D ? src[(size_t)h * D + d] : d < D + ROT ? rot[d - D] : zero;
    }
    for (int i = threadIdx.x; i < hn * VP; i += blockDim.x) {
        const int h = h0 + i / VP, d = i % VP;
        values[((page * H + h) * BC_PAGE + row) * VP + d] = d < DV ? src[(size_t)H * D + (size_t)h * DV + d] : zero;
    }
}

// One block a row.
__global__ void __launch_bounds__(128)
latent_gate_kernel(const bf16* att, const float* gate, bf16* __restrict__ out, int H, int DV, int VP) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(att); PDL_FRESH(gate);
    const size_t r = blockIdx.x;
    if (DV % 8 == 0 && VP % 8 == 0) {
        const int C = DV / 8;
        for (int i = threadIdx.x; i < H * C; i += blockDim.x) {
            const int h = i / C, d = 8 * (i - h * C);
            const float g = gate[r * H + h];
            uint4 v = *reinterpret_cast<const uint4*>(att + (r * H + h) * VP + d);
            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float lo = __uint_as_float(w[k] << 16) * g, hi = __uint_as_float(w[k] & 0xffff0000u) * g;
                const __nv_bfloat162 two = __floats2bfloat162_rn(lo, hi);
                w[k] = *reinterpret_cast<const uint32_t*>(&two);
            }
            *reinterpret_cast<uint4*>(out + r * H * DV + (size_t)h * DV + d) = v;
        }
        return;
    }
    for (int i = threadIdx.x; i < H * DV; i += blockDim.x) {
        const int h = i / DV, d = i - h * DV;
        out[r * H * DV + i] = __float2bfloat16_rn(__bfloat162float(att[(r * H + h) * VP + d]) * gate[r * H + h]);
    }
}

extern "C" int bc_latent_heads_bf16(const float* q, const float* cos_sin, int table_positions, const int* row_pos, void* out, int rows, int H, int D, int ROT,
                                    int KP, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && D > 0 && ROT >= 0 && ROT % 2 == 0 && KP >= D + ROT && (ROT == 0 || cos_sin),
                 "latent_heads: bad sizes rows=%d H=%d D=%d rot=%d padded=%d", rows, H, D, ROT, KP);
    if (rows == 0) return BC_OK;
    bc_launch(latent_heads_kernel, dim3(rows), dim3(128), 0, s, q, cos_sin, table_positions, row_pos, (bf16*)out, H, D, ROT, KP);
    BC_LAUNCH_STATUS();
}

extern "C" int bc_latent_gather_bf16(const void* c_pages, const void* r_pages, const int* page_table, const int* pg_slot, const int* pg_pos, const int* pg_last,
                                     void* ctx_c, void* ctx_r, int pages, int R, int ROT, int max_pages, int n_pages, cudaStream_t s) {
    BC_CHECK_ARG(pages >= 0 && R > 0 && R % 8 == 0 && ROT >= 0 && ROT % 8 == 0 && (ROT == 0 || (r_pages && ctx_r)),
                 "latent_gather: bad sizes pages=%d R=%d rot=%d (multiples of 8)", pages, R, ROT);
    if (pages == 0) return BC_OK;
    bc_launch(latent_gather_kernel, dim3(pages), dim3(128), 0, s, (const bf16*)c_pages, (const bf16*)r_pages, page_table, pg_slot, pg_pos, pg_last,
              (bf16*)ctx_c, (bf16*)ctx_r, R, ROT, max_pages, n_pages);
    BC_LAUNCH_STATUS();
}

extern "C" int bc_latent_spread_bf16(const void* kv, const void* ctx_r, void* keys, void* values, int rows, int H, int D, int DV, int ROT, int KP, int VP,
                                     cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && rows % BC_PAGE == 0 && H > 0 && D > 0 && DV > 0 && ROT >= 0 && KP >= D + ROT && VP >= DV && (H + LS_HEADS - 1) / LS_HEADS <= 65535,
                 "latent_spread: bad sizes rows=%d H=%d D=%d DV=%d rot=%d padded=%d, %d", rows, H, D, DV, ROT, KP, VP);
    if (rows == 0) return BC_OK;
    bc_launch(latent_spread_kernel, dim3(rows, (H + LS_HEADS - 1) / LS_HEADS), dim3(256), 0, s, (const bf16*)kv, (const bf16*)ctx_r, (bf16*)keys, (bf16*)values, H,
              D, DV, ROT, KP, VP);
    BC_LAUNCH_STATUS();
}

extern "C" int bc_latent_gate_bf16(const void* att, const float* gate, void* out, int rows, int H, int DV, int VP, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && DV > 0 && VP >= DV, "latent_gate: bad sizes rows=%d H=%d DV=%d padded=%d", rows, H, DV, VP);
    if (rows == 0) return BC_OK;
    bc_launch(latent_gate_kernel, dim3(rows), dim3(128), 0, s, (const bf16*)att, gate, (bf16*)out, H, DV, VP);
    BC_LAUNCH_STATUS();
}
