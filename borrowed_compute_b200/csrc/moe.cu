// A feed-forward of many small gated experts of which every row uses a few.
//
//   route      z = W_router h in float; score s = sigmoid(z) (or softmax over the experts); the `top` largest scores of a
//              row choose its experts (the lower index wins a tie); weights are the scores, as they are or divided by their sum
//   count, offsets, fill
//              rows sorted by expert: perm[j] = the (row, choice) pair at sorted place j, place[row * top + c] = its place,
//              and a table of tiles of MOE_BM sorted rows that lie in one expert each
//   gate_up    act[j] = silu(w g) * (w u) with g = W_gate^e x, u = W_up^e x, x the pair's row, w its weight: the weight
//              multiplies the expert's input (weight_on_input), or act[j] = silu(g) * u and the weight waits for combine
//   down       y[j] = W_down^e act[j] in float
//   combine    residual[r] += sum over r's choices, in the order of choice, of y[place] (times the weight if it waited)
//
// Every sum of a row runs in an order that the sizes alone fix, and no two blocks add into one place: a row's result is the
// same bits in any batch and at every repeat.  The products here run on the CUDA cores in float (the true 32-bit path, and
// the checked twin of the tensor-core grouped product).
#include "common.cuh"

#define MOE_BM 32
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MAX_TOP 16

// -------------------------------------------------------------------------------------- route
// Four neighbouring values of a row as floats (the row starts on a 16-byte border and k is a multiple of 4).
__device__ __forceinline__ float4 route_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 route_load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

#define ROUTE_ROWS 4        // rows a block: an expert's weights are read once for four rows
#define ROUTE_EXPERTS 8     // experts a block, one a warp

// logits[r][e] = router[e] . h[r] in float.  Block (x, y): rows 4 x .. and experts 8 y ..; a lane's share of a row's sum,
// and the order of the shares, depend on K alone, so a row's logits are the same bits in any batch.
template <class T>
__global__ void __launch_bounds__(32 * ROUTE_EXPERTS)
moe_logits_kernel(const T* __restrict__ h, const float* __restrict__ router, float* __restrict__ logits, int rows, int E, int K) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(h);
    const int r0 = blockIdx.x * ROUTE_ROWS;
    const int lane = threadIdx.x & 31, e = blockIdx.y * ROUTE_EXPERTS + (threadIdx.x >> 5);
    if (e >= E) return;
    const bool wide = K % 4 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)router % 16 == 0;
    const T* x[ROUTE_ROWS];
#pragma unroll
    for (int i = 0; i < ROUTE_ROWS; i++) x[i] = h + (size_t)min(r0 + i, rows - 1) * K;
    const float* w = router + (size_t)e * K;
    float z[ROUTE_ROWS] = {};
    if (wide) {
#pragma unroll 4
        for (int k = 4 * lane; k < K; k += 128) {           // four turns' loads are asked for together
            const float4 b = route_load4(w + k);
#pragma unroll
            for (int i = 0; i < ROUTE_ROWS; i++) {
                const float4 a = route_load4(x[i] + k);
                z[i] = fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, z[i]))));
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float b = w[k];
#pragma unroll
            for (int i = 0; i < ROUTE_ROWS; i++) z[i] = fmaf(to_f32(x[i][k]), b, z[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < ROUTE_ROWS; i++) {
        const float v = warp_sum(z[i]);
        if (lane == 0 && r0 + i < rows) logits[(size_t)(r0 + i) * E + e] = v;
    }
}

// One warp a row: the `top` largest logits (the lower index wins a tie) and their scores.
__global__ void __launch_bounds__(128)
moe_choose_kernel(const float* __restrict__ logits, const int* __restrict__ row_slot, int* __restrict__ choice, float* __restrict__ weight, int rows,
                  int E, int top, int softmax, int renorm, float factor) {
    extern __shared__ float score_all[];                    // [4][E]
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(logits);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = blockIdx.x * 4 + warp;
    if (r >= rows) return;
    if (row_slot != nullptr && row_slot[r] < 0) {           // a padding row takes no expert
        if (lane < top) {
            choice[(size_t)r * top + lane] = -1;
            weight[(size_t)r * top + lane] = 0.0f;
        }
        return;
    }
    float* score = score_all + warp * E;
    for (int e = lane; e < E; e += 32) {
        const float v = logits[(size_t)r * E + e];
        score[e] = v == v ? v : -INFINITY;                  // a row of not-a-numbers still chooses experts that exist
    }
    __syncwarp();
    // Scores from logits; the order of the experts is the order of their logits under either rule.
    float zmax = -INFINITY;
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, score[e]);
    zmax = warp_max(zmax);
    float total = 0.0f;
    if (softmax) {
        for (int e = lane; e < E; e += 32) total += expf(score[e] - zmax);
        total = warp_sum(total);
    }
    float picked_sum = 0.0f, mine = 0.0f;
    int mine_e = -1;
    for (int c = 0; c < top; c++) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float z = score[e];
            if (z != INFINITY && (best_e == 0x7fffffff || z > best)) { best = z; best_e = e; }     // taken ones are marked +inf
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7fffffff && (best_e == 0x7fffffff || ob > best || (ob == best && oe < best_e))) { best = ob; best_e = oe; }
        }
        if (best_e == 0x7fffffff) best_e = 0;
        const float s = softmax ? expf(best - zmax) / total : 1.0f / (1.0f + expf(-best));
        picked_sum += s;
        if (lane == c) { mine = s; mine_e = best_e; }
        __syncwarp();
        if (lane == 0) score[best_e] = INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        choice[(size_t)r * top + lane] = mine_e;
        // The addend keeps the division defined when every chosen score has underflowed to zero.
        weight[(size_t)r * top + lane] = (renorm ? mine / (picked_sum + 1e-20f) : mine) * factor;
    }
}

// ------------------------------------------------------------------------- sorting by expert
// One block an expert walks all (row, choice) pairs in order and counts its own.
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ choice, int pairs, int* __restrict__ counts) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(choice);
    const int e = blockIdx.x;
    int n = 0;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) n += choice[i] == e;
    const float total = block_sum((float)n, scratch);        // exact: counts stay far below 2^24
    if (threadIdx.x == 0) counts[e] = (int)total;
}

// One warp: where every expert's rows start in sorted order, and the tiles.  table: [0] the number of tiles, then for tile t
// at 1 + 3 t: expert, first sorted place, rows.  The lanes take 32 experts at a time and share their sums by shuffles.
__device__ __forceinline__ void moe_offsets_warp(const int* counts, int E, int* offsets, int* table, int max_tiles, int tile_rows) {
    const int lane = threadIdx.x & 31;
    int at = 0, tiles = 0;                                   // the same in every lane
    for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int n = e < E ? counts[e] : 0;
        const int t = (n + tile_rows - 1) / tile_rows;
        int rows_before = n, tiles_before = t;               // inclusive sums over the lanes, then made exclusive
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, rows_before, o), b = __shfl_up_sync(0xffffffffu, tiles_before, o);
            if (lane >= o) { rows_before += a; tiles_before += b; }
        }
        const int all_rows = __shfl_sync(0xffffffffu, rows_before, 31), all_tiles = __shfl_sync(0xffffffffu, tiles_before, 31);
        rows_before += at - n;
        tiles_before += tiles - t;
        if (e < E) {
            offsets[e] = rows_before;
            for (int i = 0; i < t && tiles_before + i < max_tiles; i++) {
                table[1 + 3 * (tiles_before + i)] = e;
                table[2 + 3 * (tiles_before + i)] = rows_before + i * tile_rows;
                table[3 + 3 * (tiles_before + i)] = min(tile_rows, n - i * tile_rows);
            }
        }
        at += all_rows;
        tiles += all_tiles;
    }
    if (lane == 0) {
        offsets[E] = at;
        table[0] = min(tiles, max_tiles);
    }
}

__global__ void __launch_bounds__(32) moe_offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets, int* __restrict__ table,
                                                        int max_tiles, int tile_rows) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(counts);
    moe_offsets_warp(counts, E, offsets, table, max_tiles, tile_rows);
}

// Few pairs (a step of single rows): the three kernels of the sort as one block.  A warp an expert counts, then one warp
// lays out offsets and tiles, then a warp an expert gives its pairs their places, in the order of the pairs as ever.
__global__ void __launch_bounds__(256) moe_plan_small_kernel(const int* __restrict__ choice, int pairs, int E, int tile_rows, int max_tiles,
                                                            int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ table,
                                                            int* __restrict__ perm, int* __restrict__ place) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(choice);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = warp; e < E; e += 8) {
        int n = 0;
        for (int i0 = 0; i0 < pairs; i0 += 32) n += __popc(__ballot_sync(0xffffffffu, i0 + lane < pairs && choice[i0 + lane] == e));
        if (lane == 0) counts[e] = n;
    }
    __syncthreads();
    if (warp == 0) moe_offsets_warp(counts, E, offsets, table, max_tiles, tile_rows);
    __syncthreads();
    for (int e = warp; e < E; e += 8) {
        int at = offsets[e];
        for (int i0 = 0; i0 < pairs; i0 += 32) {
            const int i = i0 + lane;
            const bool hit = i < pairs && choice[i] == e;
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int j = at + __popc(ballot & ((1u << lane) - 1u));
                perm[j] = i;
                place[i] = j;
            }
            at += __popc(ballot);
        }
    }
}

// One block an expert walks the pairs again, in the same order, and gives each of its own the next place.
__global__ void __launch_bounds__(256) moe_fill_kernel(const int* __restrict__ choice, int pairs, const int* __restrict__ offsets,
                                                      int* __restrict__ perm, int* __restrict__ place) {
    __shared__ int warp_counts[8];
    __shared__ int base;
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(choice); PDL_FRESH(offsets);
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = offsets[e];
    __syncthreads();
    for (int i0 = 0; i0 < pairs; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        const bool hit = i < pairs && choice[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_counts[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, all = 0;
        for (int w = 0; w < 8; w++) {
            if (w < warp) before += warp_counts[w];
            all += warp_counts[w];
        }
        if (hit) {
            const int j = base + before + __popc(ballot & ((1u << lane) - 1u));
            perm[j] = i;
            place[i] = j;
        }
        __syncthreads();
        if (threadIdx.x == 0) base += all;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------- grouped products
template <class T>
__device__ __forceinline__ void moe_load_tile(const T* __restrict__ src, const int* rows_of, int n_rows, int K, int k0, float (*smem)[MOE_BN + 4],
                                              int tile_rows) {
    // tile_rows x 16 values of a K-major matrix into smem[k][row]; rows_of (shared memory) names each row's source, -1: zeros.
    for (int i = threadIdx.x; i < tile_rows * 4; i += blockDim.x) {
        const int r = i >> 2, kq = (i & 3) * 4;
        const int row = r < n_rows ? rows_of[r] : -1;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + kq + j;
            smem[kq + j][r] = row >= 0 && k < K ? to_f32(src[(size_t)row * K + k]) : 0.0f;
        }
    }
}

// GATED: W is [E, 2 N, K] (gate rows, then up rows), out_act[j][n] = silu(w g) * (w u) with w = weight[perm[j]] if
// weight_on_input else 1; X rows are gathered: sorted place j reads row perm[j] / top.
// Not GATED: W is [E, N, K], X is [sorted places, K] as it lies, out_f32[j][n] = the sum.
template <class T, bool GATED>
__global__ void __launch_bounds__(128)
moe_product_kernel(const T* __restrict__ X, const T* __restrict__ W, const int* __restrict__ table, const int* __restrict__ perm,
                   const float* __restrict__ weight, T* __restrict__ out_act, float* __restrict__ out_f32, int N, int K, int top,
                   int weight_on_input) {
    __shared__ float As[MOE_BK][MOE_BN + 4];       // only MOE_BM columns used
    __shared__ float Bs[MOE_BK][MOE_BN + 4];
    __shared__ float Cs[GATED ? MOE_BK : 1][MOE_BN + 4];
    __shared__ int src_row[MOE_BM], w_row[MOE_BN];
    __shared__ float row_w[MOE_BM];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(X); PDL_FRESH(table); PDL_FRESH(perm); PDL_FRESH(weight);
    const int tile = blockIdx.y;
    if (tile >= table[0]) return;
    const int e = table[1 + 3 * tile], j0 = table[2 + 3 * tile], n_rows = table[3 + 3 * tile];
    const int n0 = blockIdx.x * MOE_BN;
    if (threadIdx.x < MOE_BM) {
        const int j = j0 + threadIdx.x;
        const bool in = threadIdx.x < n_rows;
        src_row[threadIdx.x] = !in ? -1 : GATED ? perm[j] / top : j;
        row_w[threadIdx.x] = in && GATED && weight_on_input ? weight[perm[j]] : 1.0f;
    }
    if (threadIdx.x < MOE_BN) w_row[threadIdx.x] = n0 + threadIdx.x < N ? n0 + threadIdx.x : -1;
    __syncthreads();
    const T* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;        // 16 x 8 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    float acc2[GATED ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        moe_load_tile<T>(X, src_row, n_rows, K, k0, As, MOE_BM);
        moe_load_tile<T>(We, w_row, MOE_BN, K, k0, Bs, MOE_BN);
        if (GATED) moe_load_tile<T>(We + (size_t)N * K, w_row, MOE_BN, K, k0, Cs, MOE_BN);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MOE_BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (GATED) {
                float c[4];
#pragma unroll
                for (int j = 0; j < 4; j++) c[j] = Cs[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc2[i][j] = fmaf(a[i], c[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty * 4 + i;
        if (r >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)(j0 + r) * N + n;
            if (GATED) {
                const float g = acc[i][j] * row_w[r], u = acc2[GATED ? i : 0][j] * row_w[r];
                out_act[o] = from_f32<T>(g / (1.0f + expf(-g)) * u);
            } else {
                out_f32[o] = acc[i][j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------- gather
// sorted[j] = weight[perm[j]] * x[perm[j] / top] (the weight on the expert's input) or x[perm[j] / top], for the sorted places
// j below offsets[E], the pairs that chose an expert; the places past them hold nothing that is ever written out.
template <class T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ offsets, const float* __restrict__ weight,
                  T* __restrict__ sorted, int E, int K, int top, int weight_on_input) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(x); PDL_FRESH(perm); PDL_FRESH(offsets); PDL_FRESH(weight);
    const int j = blockIdx.x;
    T* dst = sorted + (size_t)j * K;
    if (j >= offsets[E]) {
        for (int c = threadIdx.x; c < K; c += blockDim.x) dst[c] = from_f32<T>(0.0f);
        return;
    }
    const int pair = perm[j];
    const float w = weight_on_input ? weight[pair] : 1.0f;
    const T* src = x + (size_t)(pair / top) * K;
    for (int c = threadIdx.x; c < K; c += blockDim.x) dst[c] = from_f32<T>(w * to_f32(src[c]));
}

// ------------------------------------------------------------------------------------ combine
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ choice, const int* __restrict__ place, const float* __restrict__ weight,
                   float* __restrict__ residual, int E, int top, int weight_on_output) {
    __shared__ int where[MOE_MAX_TOP];
    __shared__ float factor[MOE_MAX_TOP];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(y); PDL_FRESH(choice); PDL_FRESH(place); PDL_FRESH(weight);
    const int r = blockIdx.x;
    // The row's places first, so that the loads of a column's values do not each wait for one.
    if ((int)threadIdx.x < top) {
        const bool chosen = choice[(size_t)r * top + threadIdx.x] >= 0;
        where[threadIdx.x] = chosen ? place[(size_t)r * top + threadIdx.x] : -1;
        factor[threadIdx.x] = weight_on_output ? weight[(size_t)r * top + threadIdx.x] : 1.0f;
    }
    __syncthreads();
    bool any = false;
    for (int i = 0; i < top; i++) any = any || where[i] >= 0;
    if (!any) return;
    if (E % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)residual % 16 == 0) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
            for (int i = 0; i < top; i++) {
                if (where[i] < 0) continue;
                const float4 v = *reinterpret_cast<const float4*>(y + (size_t)where[i] * E + c);
                const float f = factor[i];
                sum = weight_on_output ? make_float4(fmaf(f, v.x, sum.x), fmaf(f, v.y, sum.y), fmaf(f, v.z, sum.z), fmaf(f, v.w, sum.w))
                                       : make_float4(sum.x + v.x, sum.y + v.y, sum.z + v.z, sum.w + v.w);
            }
            float4* out = reinterpret_cast<float4*>(residual + (size_t)r * E + c);
            const float4 old = *out;
            *out = make_float4(old.x + sum.x, old.y + sum.y, old.z + sum.z, old.w + sum.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        float sum = 0.0f;
#pragma unroll 4
        for (int i = 0; i < top; i++) {
            if (where[i] < 0) continue;
            const float v = y[(size_t)where[i] * E + c];
            sum = weight_on_output ? fmaf(factor[i], v, sum) : sum + v;
        }
        residual[(size_t)r * E + c] += sum;
    }
}

// ------------------------------------------------------------------------------------ launchers
template <class T>
static int route(const void* h, const float* router, const int* row_slot, float* logits, int* choice, float* weight, int rows, int E, int K, int top,
                 int softmax, int renorm, float factor, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0 && K > 0 && top > 0 && top <= E && top <= MOE_MAX_TOP && E <= 2048, "moe_route: bad sizes rows=%d E=%d K=%d top=%d", rows, E, K, top);
    if (rows == 0) return BC_OK;
    const int groups = (E + ROUTE_EXPERTS - 1) / ROUTE_EXPERTS;
    BC_CHECK_ARG(groups <= 65535, "moe_route: too many experts (%d)", E);
    bc_launch(moe_logits_kernel<T>, dim3((rows + ROUTE_ROWS - 1) / ROUTE_ROWS, groups), dim3(32 * ROUTE_EXPERTS), 0, s, (const T*)h, router, logits, rows, E, K);
    bc_launch(moe_choose_kernel, dim3((rows + 3) / 4), dim3(128), (size_t)4 * E * sizeof(float), s, (const float*)logits, row_slot, choice, weight, rows,
              E, top, softmax, renorm, factor);
    BC_LAUNCH_STATUS();
}
// h: [rows, K] of the activation type; router: [E, K] float; row_slot: [rows] (negative: a padding row; may be null);
// logits: [rows, E] float (scratch); choice: [rows, top] int; weight: [rows, top] float, every weight times `factor`.
extern "C" int bc_moe_route_f32(const void* h, const float* router, const int* row_slot, float* logits, int* choice, float* weight, int rows, int E,
                                int K, int top, int softmax, int renorm, float factor, cudaStream_t s) {
    return route<float>(h, router, row_slot, logits, choice, weight, rows, E, K, top, softmax, renorm, factor, s);
}
extern "C" int bc_moe_route_bf16(const void* h, const float* router, const int* row_slot, float* logits, int* choice, float* weight, int rows, int E,
                                 int K, int top, int softmax, int renorm, float factor, cudaStream_t s) {
    return route<bf16>(h, router, row_slot, logits, choice, weight, rows, E, K, top, softmax, renorm, factor, s);
}

extern "C" int bc_moe_max_tiles(int pairs, int E, int tile_rows) { return (pairs + tile_rows - 1) / tile_rows + E; }
extern "C" int bc_moe_simt_tile_rows() { return MOE_BM; }

// choice: [pairs]; counts: [E]; offsets: [E + 1]; table: [1 + 3 * bc_moe_max_tiles(pairs, E, tile_rows)]; perm, place: [pairs].
extern "C" int bc_moe_plan(const int* choice, int pairs, int E, int tile_rows, int* counts, int* offsets, int* table, int* perm, int* place,
                           cudaStream_t s) {
    BC_CHECK_ARG(pairs >= 0 && E > 0 && E <= 65535 && tile_rows > 0, "moe_plan: bad sizes pairs=%d E=%d tile_rows=%d", pairs, E, tile_rows);
    if (pairs == 0) return BC_OK;
    if (pairs <= 1024 && E <= 1024) {      // by the sizes alone
        bc_launch(moe_plan_small_kernel, dim3(1), dim3(256), 0, s, choice, pairs, E, tile_rows, bc_moe_max_tiles(pairs, E, tile_rows), counts, offsets,
                  table, perm, place);
        BC_LAUNCH_STATUS();
    }
    bc_launch(moe_count_kernel, dim3(E), dim3(256), 0, s, choice, pairs, counts);
    bc_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, s, (const int*)counts, E, offsets, table, bc_moe_max_tiles(pairs, E, tile_rows), tile_rows);
    bc_launch(moe_fill_kernel, dim3(E), dim3(256), 0, s, choice, pairs, (const int*)offsets, perm, place);
    BC_LAUNCH_STATUS();
}

template <class T>
static int products(int gated, const void* X, const void* W, const int* table, const int* perm, const float* weight, void* out, int pairs, int E,
                    int N, int K, int top, int weight_on_input, cudaStream_t s) {
    BC_CHECK_ARG(pairs >= 0 && E > 0 && N > 0 && K > 0 && top > 0, "moe_product: bad sizes pairs=%d E=%d N=%d K=%d", pairs, E, N, K);
    if (pairs == 0) return BC_OK;
    const int tiles = bc_moe_max_tiles(pairs, E, MOE_BM);
    BC_CHECK_ARG(tiles <= 65535, "moe_product: %d tiles are too many", tiles);
    dim3 grid((N + MOE_BN - 1) / MOE_BN, tiles);
    if (gated)
        bc_launch(moe_product_kernel<T, true>, grid, dim3(128), 0, s, (const T*)X, (const T*)W, table, perm, weight, (T*)out, (float*)nullptr, N, K,
                  top, weight_on_input);
    else
        bc_launch(moe_product_kernel<T, false>, grid, dim3(128), 0, s, (const T*)X, (const T*)W, table, perm, weight, (T*)nullptr, (float*)out, N, K,
                  top, 0);
    BC_LAUNCH_STATUS();
}
// gated: X [rows, K], W [E, 2 N, K], out [pairs, N] of the activation type; else X [pairs, K], W [E, N, K], out [pairs, N] float.
extern "C" int bc_moe_product_f32(int gated, const void* X, const void* W, const int* table, const int* perm, const float* weight, void* out,
                                  int pairs, int E, int N, int K, int top, int weight_on_input, cudaStream_t s) {
    return products<float>(gated, X, W, table, perm, weight, out, pairs, E, N, K, top, weight_on_input, s);
}
extern "C" int bc_moe_product_bf16(int gated, const void* X, const void* W, const int* table, const int* perm, const float* weight, void* out,
                                   int pairs, int E, int N, int K, int top, int weight_on_input, cudaStream_t s) {
    return products<bf16>(gated, X, W, table, perm, weight, out, pairs, E, N, K, top, weight_on_input, s);
}

template <class T>
static int gather(const void* x, const int* perm, const int* offsets, const float* weight, void* sorted, int pairs, int E, int K, int top,
                  int weight_on_input, cudaStream_t s) {
    BC_CHECK_ARG(pairs >= 0 && E > 0 && K > 0 && top > 0, "moe_gather: bad sizes pairs=%d E=%d K=%d top=%d", pairs, E, K, top);
    if (pairs == 0) return BC_OK;
    bc_launch(moe_gather_kernel<T>, dim3(pairs), dim3(K >= 2048 ? 256 : 128), 0, s, (const T*)x, perm, offsets, weight, (T*)sorted, E, K, top, weight_on_input);
    BC_LAUNCH_STATUS();
}
// x: [rows, K]; sorted: [pairs, K]; perm: [pairs]; offsets: [E + 1]; weight: [pairs] in the order of (row, choice).
extern "C" int bc_moe_gather_f32(const void* x, const int* perm, const int* offsets, const float* weight, void* sorted, int pairs, int E, int K,
                                 int top, int weight_on_input, cudaStream_t s) {
    return gather<float>(x, perm, offsets, weight, sorted, pairs, E, K, top, weight_on_input, s);
}
extern "C" int bc_moe_gather_bf16(const void* x, const int* perm, const int* offsets, const float* weight, void* sorted, int pairs, int E, int K,
                                  int top, int weight_on_input, cudaStream_t s) {
    return gather<bf16>(x, perm, offsets, weight, sorted, pairs, E, K, top, weight_on_input, s);
}

// y: [pairs, width] float in sorted order; residual: [rows, width] float.
extern "C" int bc_moe_combine(const float* y, const int* choice, const int* place, const float* weight, float* residual, int rows, int width, int top,
                              int weight_on_output, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && width > 0 && top > 0, "moe_combine: bad sizes rows=%d width=%d top=%d", rows, width, top);
    if (rows == 0) return BC_OK;
    bc_launch(moe_combine_kernel, dim3(rows), dim3(width >= 1024 ? 256 : 128), 0, s, y, choice, place, weight, residual, width, top, weight_on_output);
    BC_LAUNCH_STATUS();
}
