// Latent attention for steps of one row a sequence, bf16: the cached positions split across blocks, sixteen heads
// sharing every read of the cache.
//
// A position keeps one vector c (R values) and, if the mixer rotates, one rotated key part r (ROT values); every head's
// key is a product of c (moved to the query's side: a_n = [Wuk_n^T q_n | rot(qr_n)]) and its value a product of the sum
// over positions of p c, so all heads read the same R + ROT values a position and attention is
//     S = A [heads, R + ROT] x [c | r]^T [R + ROT, positions],  P = softmax(S * scale),  O = P x c [positions, R].
// A block takes (row, sixteen heads, split of the positions).  The sixteen heads are the rows of m16n8k16 tensor-core
// tiles.  Pages of 64 positions stream through two stages of shared memory by cp.async as rows [c | r | 0 .. 0] of a
// multiple of sixteen values, padded by eight so that eight rows fall into eight different banks.  Of a page, each of
// the eight warps takes eight positions for S (so the page's keys are multiplied once; eight warps, because one warp a
// scheduler has nothing to hide its own latencies behind), the running maximum is the block's (through shared memory),
// P goes to shared memory as bf16, and each warp takes every eighth pair of eight value columns for O (so the
// accumulators, 16 x R floats, are spread over the warps).  With one split the block divides and
// writes; with several every block leaves (maximum, sum, O) in scratch memory and a second kernel merges them in the
// order of the splits.  Nothing of the launch depends on the lengths, which are read on the device, so a captured graph
// serves every step.  Sums run in an order that the sizes and the number of splits fix.
#include "common.cuh"
#include "mma_tiles.cuh"

#define LD_THREADS 256
#define LD_WARPS (LD_THREADS / 32)
#define LD_STAGES 2
#define LD_HEADS 16
#define LD_PS 72            // a row of P in shared memory: 64 positions and eight of padding

__host__ __device__ __forceinline__ int ld_up16(int n) { return (n + 15) & ~15; }
// Floats one (row, group of heads, split) leaves in scratch memory: 16 maxima, 16 sums, 16 rows of O.
__host__ __device__ __forceinline__ size_t ld_partial_floats(int R) { return 32 + (size_t)LD_HEADS * ld_up16(R); }

// MAXP: pairs of eight value columns a warp may own (R <= 128 MAXP).
template <int MAXP>
__global__ void __launch_bounds__(LD_THREADS)
latent_decode_kernel(const bf16* a, const bf16* c_pages, const bf16* r_pages, const int* __restrict__ page_table, const int* __restrict__ row_pos,
                     const int* __restrict__ row_slot, bf16* __restrict__ out, float* __restrict__ scratch, int H, int R, int ROT, int max_pages,
                     int n_pages, int window, float scale_log2, int splits, const float* __restrict__ sink) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int W = R + ROT, KW = ld_up16(W), KWS = KW + 8, CH = KW / 8, RP = ld_up16(R), NPAIR = RP / 16;
    bf16* As = reinterpret_cast<bf16*>(smem);                 // [16][KWS]
    bf16* tiles = As + LD_HEADS * KWS;                         // LD_STAGES x [64][KWS]
    bf16* Ps = tiles + (size_t)LD_STAGES * BC_PAGE * KWS;      // [16][LD_PS]
    float* wmax = reinterpret_cast<float*>(Ps + LD_HEADS * LD_PS);   // [4][16]
    float* lsum = wmax + LD_WARPS * LD_HEADS;                  // [LD_WARPS][16]

    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(a); PDL_FRESH(c_pages); PDL_FRESH(r_pages);
    const int r = blockIdx.x, hg = blockIdx.y, z = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3, j4 = lane >> 3, r8 = lane & 7;
    const int slot = row_slot[r];
    if (slot < 0) {
        // A row of no sequence: zeros where one split writes the result; the merge of several writes them itself.
        if (splits == 1)
            for (int i = threadIdx.x; i < LD_HEADS * R; i += LD_THREADS) {
                const int head = hg * LD_HEADS + i / R;
                if (head < H) out[((size_t)r * H + head) * R + i % R] = __float2bfloat16_rn(0.0f);
            }
        return;
    }
    const int pos = row_pos[r];
    const int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    const int* pages = page_table + (size_t)slot * max_pages;
    const int t_begin = lo / BC_PAGE, t_end = pos / BC_PAGE + 1;
    const int per = (t_end - t_begin + splits - 1) / splits;
    const int my_begin = t_begin + z * per;
    const int n_tiles = max(0, min(t_end, my_begin + per) - my_begin);

    // The sixteen heads' absorbed queries, rows of heads past the last and columns past R + ROT zero.
    for (int i = threadIdx.x; i < LD_HEADS * CH; i += LD_THREADS) {
        const int row = i / CH, c = i - row * CH, head = hg * LD_HEADS + row;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head < H && c * 8 < W) v = *reinterpret_cast<const uint4*>(a + ((size_t)r * H + head) * W + c * 8);
        *reinterpret_cast<uint4*>(As + (size_t)row * KWS + c * 8) = v;
    }
    auto page_of = [&](int tile) {
        const int page = tile < max_pages ? pages[tile] : -1;
        return page >= 0 && page < n_pages ? page : -1;
    };
    auto load_tile = [&](int tile, int stage) {
        const int page = page_of(tile);
        if (page < 0) return;
        bf16* dst = tiles + (size_t)stage * BC_PAGE * KWS;
        const bf16* cs = c_pages + (size_t)page * BC_PAGE * R;
        const bf16* rs = r_pages + (size_t)page * BC_PAGE * ROT;
        // A lane keeps its columns (sixteen bytes each, neighbours in a row for neighbouring lanes) and a warp every fourth row:
        // no division in the loop, which one warp a scheduler issues with nothing to hide behind.
        for (int c = lane; c < CH; c += 32) {
            const int col = c * 8;
            bf16* d = dst + col;
            if (col < R) {
                const bf16* src = cs + col;
#pragma unroll 4
                for (int row = warp; row < BC_PAGE; row += LD_THREADS / 32) cp_async16(ad_smem(d + (size_t)row * KWS), src + (size_t)row * R);
            } else if (col < W) {
                const bf16* src = rs + (col - R);
#pragma unroll 4
                for (int row = warp; row < BC_PAGE; row += LD_THREADS / 32) cp_async16(ad_smem(d + (size_t)row * KWS), src + (size_t)row * ROT);
            } else {
                for (int row = warp; row < BC_PAGE; row += LD_THREADS / 32) *reinterpret_cast<uint4*>(d + (size_t)row * KWS) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    float o[MAXP][2][4];
#pragma unroll
    for (int i = 0; i < MAXP; i++)
#pragma unroll
        for (int j = 0; j < 2; j++) o[i][j][0] = o[i][j][1] = o[i][j][2] = o[i][j][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    if (n_tiles > 0) load_tile(my_begin, 0);
    cp_async_commit();
    const uint32_t a_base = ad_smem(As), p_base = ad_smem(Ps);
    for (int it = 0; it < n_tiles; it++) {
        cp_async_wait<0>();
        __syncthreads();
        if (it + 1 < n_tiles) load_tile(my_begin + it + 1, (it + 1) % LD_STAGES);
        cp_async_commit();
        const int tile = my_begin + it;
        if (page_of(tile) < 0) continue;
        bf16* tp = tiles + (size_t)(it % LD_STAGES) * BC_PAGE * KWS;
        const uint32_t t_base = ad_smem(tp);
        if (tile == pos / BC_PAGE && pos % BC_PAGE != BC_PAGE - 1) {
            // What lies past the row's own position in its page belongs to nobody (another sequence that held the page may
            // have left not-a-numbers, and 0 x NaN is NaN in the product with the values): cleared in the copy.
            const int first = pos % BC_PAGE + 1;
            for (int i = threadIdx.x; i < (BC_PAGE - first) * CH; i += LD_THREADS)
                *reinterpret_cast<uint4*>(tp + (size_t)(first + i / CH) * KWS + (i % CH) * 8) = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
        }
        // S for the sixteen heads against this warp's sixteen positions of the page.
        // S for the sixteen heads against this warp's eight positions of the page.  One load brings the eight positions' values
        // of two steps; the even and the odd steps add into sets of their own (two chains of products side by side), which
        // are added at the end, in an order the sizes fix.
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int k_steps = KW / 16;
        for (int kd = 0; kd < k_steps; kd += 2) {
            uint32_t af[4], b0, b1, b2, b3;
            // Past the last step of an odd count the load reads the row's padding and the start of the next row (inside shared
            // memory); those two registers are not used.
            ldmatrix_x4(t_base + ((8 * warp + r8) * KWS + (kd * 2 + j4) * 8) * 2, b0, b1, b2, b3);
            ldmatrix_x4(a_base + ((r8 + 8 * (j4 & 1)) * KWS + (kd * 2 + (j4 >> 1)) * 8) * 2, af[0], af[1], af[2], af[3]);
            mma_16816(s, af, b0, b1);
            if (kd + 1 < k_steps) {
                ldmatrix_x4(a_base + ((r8 + 8 * (j4 & 1)) * KWS + ((kd + 1) * 2 + (j4 >> 1)) * 8) * 2, af[0], af[1], af[2], af[3]);
                mma_16816(s_odd, af, b2, b3);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) s[e] += s_odd[e];
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int t = tile * BC_PAGE + 8 * warp + 2 * tq + (e & 1);
            s[e] = t >= lo && t <= pos ? s[e] * scale_log2 : -INFINITY;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], s[e]);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            if (tq == 0) wmax[warp * LD_HEADS + gq + 8 * i] = tmax[i];
        }
        __syncthreads();
        float corr[2], base[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int row = gq + 8 * i;
            float tm = wmax[row];
#pragma unroll
            for (int w = 1; w < LD_WARPS; w++) tm = fmaxf(tm, wmax[w * LD_HEADS + row]);
            const float mn = fmaxf(m[i], tm);
            corr[i] = mn == -INFINITY ? 1.0f : fast_exp2(m[i] - mn);
            base[i] = mn == -INFINITY ? 0.0f : mn;
            m[i] = mn;
        }
        float psum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            s[e] = fast_exp2(s[e] - base[e >> 1]);
            psum[e >> 1] += s[e];
        }
        {
            const int col = 8 * warp + 2 * tq;
            *reinterpret_cast<uint32_t*>(Ps + (size_t)gq * LD_PS + col) = pack_bf16(s[0], s[1]);
            *reinterpret_cast<uint32_t*>(Ps + (size_t)(gq + 8) * LD_PS + col) = pack_bf16(s[2], s[3]);
        }
        l[0] = l[0] * corr[0] + psum[0];
        l[1] = l[1] * corr[1] + psum[1];
        __syncthreads();
        // O += P c for this warp's value columns.
#pragma unroll
        for (int jp = 0; jp < MAXP; jp++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                o[jp][j][0] *= corr[0]; o[jp][j][1] *= corr[0]; o[jp][j][2] *= corr[1]; o[jp][j][3] *= corr[1];
            }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            uint32_t pf[4];
            ldmatrix_x4(p_base + ((r8 + 8 * (j4 & 1)) * LD_PS + (kk * 2 + (j4 >> 1)) * 8) * 2, pf[0], pf[1], pf[2], pf[3]);
#pragma unroll
            for (int jp = 0; jp < MAXP; jp++) {
                const int pair = warp + LD_WARPS * jp;
                if (pair < NPAIR) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(t_base + ((kk * 16 + (j4 & 1) * 8 + r8) * KWS + (2 * pair + (j4 >> 1)) * 8) * 2, b0, b1, b2, b3);
                    mma_16816(o[jp][0], pf, b0, b1);
                    mma_16816(o[jp][1], pf, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (tq == 0) lsum[warp * LD_HEADS + gq + 8 * i] = l[i];
    }
    __syncthreads();
    float total[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int row = gq + 8 * i;
        float t = lsum[row];
#pragma unroll
        for (int w = 1; w < LD_WARPS; w++) t += lsum[w * LD_HEADS + row];
        total[i] = t;
    }
    if (splits == 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int head = hg * LD_HEADS + gq + 8 * i;
            if (head >= H) continue;
            // A sink is one more term of the row's sum, e^(the head's number) against the row's maximum, with no key and no value.
            if (sink != nullptr && m[i] != -INFINITY) total[i] += fast_exp2(sink[head] * 1.4426950408889634f - m[i]);
            const float inv = total[i] > 0.0f ? 1.0f / total[i] : 0.0f;
            bf16* dst = out + ((size_t)r * H + head) * R;
#pragma unroll
            for (int jp = 0; jp < MAXP; jp++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int d = (warp + LD_WARPS * jp) * 16 + j * 8 + 2 * tq;
                    if (d < R) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[jp][j][2 * i] * inv, o[jp][j][2 * i + 1] * inv);
                }
        }
        return;
    }
    float* part = scratch + (((size_t)r * gridDim.y + hg) * splits + z) * ld_partial_floats(R);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int row = gq + 8 * i;
        if (warp == 0 && tq == 0) {
            part[row] = m[i];
            part[LD_HEADS + row] = total[i];
        }
#pragma unroll
        for (int jp = 0; jp < MAXP; jp++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int d = (warp + LD_WARPS * jp) * 16 + j * 8 + 2 * tq;
                if (d < RP) *reinterpret_cast<float2*>(part + 32 + (size_t)row * RP + d) = make_float2(o[jp][j][2 * i], o[jp][j][2 * i + 1]);
            }
    }
}

// One block a (row, head): the splits' partial results in their order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* scratch, const int* __restrict__ row_slot, bf16* __restrict__ out, int H, int R, int groups, int splits,
                    const float* __restrict__ sink) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(scratch);
    const int r = blockIdx.x, h = blockIdx.y, hg = h / LD_HEADS, row = h % LD_HEADS;
    const int RP = ld_up16(R);
    bf16* dst = out + ((size_t)r * H + h) * R;
    const float* part = scratch + ((size_t)r * groups + hg) * splits * ld_partial_floats(R);
    // The splits' maxima once, in shared memory (a split's number is the thread's), then their weights; every thread adds its
    // columns over the splits in their order, four columns side by side so that the loads of a split overlap (R <= 512: at
    // most four columns a thread).
    __shared__ float wz[64], lz[64];
    const bool live = row_slot[r] >= 0;
    if (threadIdx.x < 64) wz[threadIdx.x] = live && threadIdx.x < splits ? part[(size_t)threadIdx.x * ld_partial_floats(R) + row] : -INFINITY;
    else lz[threadIdx.x - 64] = live && threadIdx.x - 64 < splits ? part[(size_t)(threadIdx.x - 64) * ld_partial_floats(R) + LD_HEADS + row] : 0.0f;
    __syncthreads();
    float top = -INFINITY;
    for (int z = 0; z < splits; z++) top = fmaxf(top, wz[z]);
    if (top == -INFINITY) {
        for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = __float2bfloat16_rn(0.0f);
        return;
    }
    __syncthreads();
    if (threadIdx.x < 64) wz[threadIdx.x] = fast_exp2(wz[threadIdx.x] - top);
    __syncthreads();
    float total = 0.0f;
    for (int z = 0; z < splits; z++) total += wz[z] * lz[z];
    if (sink != nullptr) total += fast_exp2(sink[h] * 1.4426950408889634f - top);      // the sink's term, once a row
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 2
    for (int z = 0; z < splits; z++) {
        const float w = wz[z];
        const float* p = part + (size_t)z * ld_partial_floats(R) + 32 + (size_t)row * RP;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int d = threadIdx.x + 128 * k;
            const float v = (w > 0.0f && d < R) ? p[d] : 0.0f;      // a split that saw nothing may hold anything
            acc[k] = fmaf(w, v, acc[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int d = threadIdx.x + 128 * k;
        if (d < R) dst[d] = __float2bfloat16_rn(acc[k] * inv);
    }
}

extern "C" int bc_latent_decode_accepts(int H, int R, int ROT) {
    return H > 0 && R > 0 && R % 8 == 0 && ROT >= 0 && ROT % 8 == 0 && R <= 512 && ROT <= 128;
}

static size_t ld_smem_bytes(int R, int ROT) {
    const int KWS = ld_up16(R + ROT) + 8;
    return (size_t)(LD_HEADS + LD_STAGES * BC_PAGE) * KWS * 2 + LD_HEADS * LD_PS * 2 + 2 * LD_WARPS * LD_HEADS * sizeof(float);
}

extern "C" long long bc_latent_decode_scratch_floats(int rows, int H, int R, int splits) {
    return splits <= 1 ? 0 : (long long)rows * ((H + LD_HEADS - 1) / LD_HEADS) * splits * (long long)ld_partial_floats(R);
}

template <int MAXP>
static int decode_launch(const void* a, const void* c_pages, const void* r_pages, const int* page_table, const int* row_pos, const int* row_slot, void* out,
                         float* scratch, int rows, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale, int splits, const float* sink,
                         cudaStream_t s) {
    const size_t smem = ld_smem_bytes(R, ROT);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(latent_decode_kernel<MAXP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            bc_set_error("latent_decode: cannot set shared memory to %zu: %s", smem, cudaGetErrorString(e));
            return (int)e;
        }
        configured = smem;
    }
    const int groups = (H + LD_HEADS - 1) / LD_HEADS;
    cudaError_t e = bc_launch(latent_decode_kernel<MAXP>, dim3(rows, groups, splits), dim3(LD_THREADS), smem, s, (const bf16*)a, (const bf16*)c_pages,
                              (const bf16*)r_pages, page_table, row_pos, row_slot, (bf16*)out, scratch, H, R, ROT, max_pages, n_pages, window,
                              scale * 1.4426950408889634f, splits, sink);
    if (e != cudaSuccess) {
        bc_set_error("latent_decode: %s", cudaGetErrorString(e));
        return (int)e;
    }
    if (splits > 1) bc_launch(latent_merge_kernel, dim3(rows, H), dim3(128), 0, s, (const float*)scratch, row_slot, (bf16*)out, H, R, groups, splits, sink);
    BC_LAUNCH_STATUS();
}

extern "C" int bc_latent_decode_bf16(const void* a, const void* c_pages, const void* r_pages, const int* page_table, const int* row_pos, const int* row_slot,
                                     void* out, float* scratch, int rows, int H, int R, int ROT, int max_pages, int n_pages, int window, float scale,
                                     int splits, const float* sink, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && bc_latent_decode_accepts(H, R, ROT) && window >= 0 && splits >= 1 && splits <= 64 && H <= 16 * 65535,
                 "latent_decode: bad sizes rows=%d H=%d R=%d rot=%d splits=%d (latents in multiples of 8 up to 512, rotated parts up to 128, at most 64 splits)", rows, H, R, ROT,
                 splits);
    BC_CHECK_ARG((ROT == 0 || r_pages) && (splits == 1 || scratch), "latent_decode: rotated keys or scratch memory missing");
    if (rows == 0) return BC_OK;
    if (R <= 128) return decode_launch<1>(a, c_pages, r_pages, page_table, row_pos, row_slot, out, scratch, rows, H, R, ROT, max_pages, n_pages, window, scale, splits, sink, s);
    if (R <= 256) return decode_launch<2>(a, c_pages, r_pages, page_table, row_pos, row_slot, out, scratch, rows, H, R, ROT, max_pages, n_pages, window, scale, splits, sink, s);
    return decode_launch<4>(a, c_pages, r_pages, page_table, row_pos, row_slot, out, scratch, rows, H, R, ROT, max_pages, n_pages, window, scale, splits, sink, s);
}
