// Kernels for blocks that norm a sublayer's result before it joins the float residual stream, and for feed-forwards
// whose activation is the square of relu.
//
//   norm_add     x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w          (y float: the sublayer's result)
//   norm_add_norm   the same, then h[r] = x[r] / sqrt(mean(x[r]^2) + eps2) * w2 in the activation type for the sublayer that
//                follows, and y[r] = 0 for its result: one kernel between the two sublayers of a block
//   relu2        out = max(z, 0)^2 in the activation type               (z float: an up product)
//   glu_clipped  out = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit), from z = [g | u] float
//   gated_add    x[r] += sigmoid(g . h[r]) * y[r]                       (one number a row: a gate on a shared expert)
//   table_route  choice[r] = table[token[r]], weight = 1 / top         (experts named by the token id, no router)
//
// A row's sums run in an order that its width alone fixes.
#include "common.cuh"

__global__ void norm_add_kernel(const float* y, const float* __restrict__ w, float* x, int E, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(y); PDL_FRESH(x);
    const float* yr = y + (size_t)blockIdx.x * E;
    float* xr = x + (size_t)blockIdx.x * E;
    float s = 0.0f;
    if (E % 4 == 0) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(yr + c);
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        s = block_sum(s, scratch);
        const float f = 1.0f / sqrtf(s / (float)E + eps);
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(yr + c);
            const float4 g = *reinterpret_cast<const float4*>(w + c);
            float4 o = *reinterpret_cast<float4*>(xr + c);
            o.x += v.x * f * g.x; o.y += v.y * f * g.y; o.z += v.z * f * g.z; o.w += v.w * f * g.w;
            *reinterpret_cast<float4*>(xr + c) = o;
        }
        return;
    }
    for (int c = threadIdx.x; c < E; c += blockDim.x) s += yr[c] * yr[c];
    s = block_sum(s, scratch);
    const float f = 1.0f / sqrtf(s / (float)E + eps);
    for (int c = threadIdx.x; c < E; c += blockDim.x) xr[c] += yr[c] * f * w[c];
}

static int pick(int n) { int t = 32; while (t < n && t < 256) t *= 2; return t; }

// y: [rows, E] float; w: [E] float; x: [rows, E] float, changed in place.
extern "C" int bc_norm_add_f32(const float* y, const float* w, float* x, int rows, int E, float eps, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0 && eps > 0.0f, "norm_add: bad sizes rows=%d E=%d eps=%g", rows, E, (double)eps);
    if (rows == 0) return BC_OK;
    bc_launch(norm_add_kernel, dim3(rows), dim3(pick(E % 4 == 0 ? E / 4 : E)), 0, s, y, w, x, E, eps);
    BC_LAUNCH_STATUS();
}

// A thread keeps its columns through both norms: it adds into x the columns whose squares it then sums.
template <class T>
__global__ void norm_add_norm_kernel(float* y, const float* __restrict__ wb, float* x, const float* __restrict__ w2, T* __restrict__ h, int E, float eps_b,
                                     float eps_2) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(y); PDL_FRESH(x);
    float* yr = y + (size_t)blockIdx.x * E;
    float* xr = x + (size_t)blockIdx.x * E;
    T* hr = h + (size_t)blockIdx.x * E;
    float s = 0.0f, t = 0.0f;
    if (E % 4 == 0) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(yr + c);
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        s = block_sum(s, scratch);
        const float f = 1.0f / sqrtf(s / (float)E + eps_b);
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(yr + c);
            const float4 g = *reinterpret_cast<const float4*>(wb + c);
            float4 o = *reinterpret_cast<float4*>(xr + c);
            o.x += v.x * f * g.x; o.y += v.y * f * g.y; o.z += v.z * f * g.z; o.w += v.w * f * g.w;
            *reinterpret_cast<float4*>(xr + c) = o;
            *reinterpret_cast<float4*>(yr + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            t += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
        }
        t = block_sum(t, scratch);
        const float f2 = 1.0f / sqrtf(t / (float)E + eps_2);
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 o = *reinterpret_cast<const float4*>(xr + c);
            const float4 g = *reinterpret_cast<const float4*>(w2 + c);
            hr[c] = from_f32<T>(o.x * f2 * g.x); hr[c + 1] = from_f32<T>(o.y * f2 * g.y);
            hr[c + 2] = from_f32<T>(o.z * f2 * g.z); hr[c + 3] = from_f32<T>(o.w * f2 * g.w);
        }
        return;
    }
    for (int c = threadIdx.x; c < E; c += blockDim.x) s += yr[c] * yr[c];
    s = block_sum(s, scratch);
    const float f = 1.0f / sqrtf(s / (float)E + eps_b);
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        const float o = xr[c] + yr[c] * f * wb[c];
        xr[c] = o;
        yr[c] = 0.0f;
        t += o * o;
    }
    t = block_sum(t, scratch);
    const float f2 = 1.0f / sqrtf(t / (float)E + eps_2);
    for (int c = threadIdx.x; c < E; c += blockDim.x) hr[c] = from_f32<T>(xr[c] * f2 * w2[c]);
}

// y: [rows, E] float, left as zeros; wb, w2: [E] float; x: [rows, E] float, changed in place; h: [rows, E] of the activation type.
template <class T> static int norm_add_norm(float* y, const float* wb, float* x, const float* w2, void* h, int rows, int E, float eps_b, float eps_2, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0 && eps_b > 0.0f && eps_2 > 0.0f, "norm_add_norm: bad sizes rows=%d E=%d eps=%g, %g", rows, E, (double)eps_b, (double)eps_2);
    if (rows == 0) return BC_OK;
    bc_launch(norm_add_norm_kernel<T>, dim3(rows), dim3(pick(E % 4 == 0 ? E / 4 : E)), 0, s, y, wb, x, w2, (T*)h, E, eps_b, eps_2);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_norm_add_norm_f32(float* y, const float* wb, float* x, const float* w2, void* h, int rows, int E, float eps_b, float eps_2, cudaStream_t s) {
    return norm_add_norm<float>(y, wb, x, w2, h, rows, E, eps_b, eps_2, s);
}
extern "C" int bc_norm_add_norm_bf16(float* y, const float* wb, float* x, const float* w2, void* h, int rows, int E, float eps_b, float eps_2, cudaStream_t s) {
    return norm_add_norm<bf16>(y, wb, x, w2, h, rows, E, eps_b, eps_2, s);
}

template <class T>
__global__ void relu2_kernel(const float* z, T* __restrict__ out, size_t n) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(z);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(z[i], 0.0f);
        out[i] = from_f32<T>(v * v);
    }
}
template <class T> static int relu2(const float* z, void* out, long long n, cudaStream_t s) {
    BC_CHECK_ARG(n >= 0, "relu2: bad size %lld", n);
    if (n == 0) return BC_OK;
    const long long blocks = (n + 255) / 256;
    bc_launch(relu2_kernel<T>, dim3((unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(256), 0, s, z, (T*)out, (size_t)n);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_relu2_f32(const float* z, void* out, long long n, cudaStream_t s) { return relu2<float>(z, out, n, s); }
extern "C" int bc_relu2_bf16(const float* z, void* out, long long n, cudaStream_t s) { return relu2<bf16>(z, out, n, s); }

// z: [rows, 2 F] float, the gate's sums then the up sums of a row; out: [rows, F].
template <class T>
__global__ void glu_clipped_kernel(const float* z, T* __restrict__ out, int F, size_t n, float limit, float alpha) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(z);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / F;
        const int j = (int)(i - r * F);
        const float g = fminf(z[r * 2 * F + j], limit);
        const float u = fminf(fmaxf(z[r * 2 * F + F + j], -limit), limit);
        out[i] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}
template <class T> static int glu_clipped(const float* z, void* out, int rows, int F, float limit, float alpha, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && F > 0 && limit > 0.0f, "glu_clipped: bad sizes rows=%d F=%d limit=%g", rows, F, (double)limit);
    const long long n = (long long)rows * F;
    if (n == 0) return BC_OK;
    const long long blocks = (n + 255) / 256;
    bc_launch(glu_clipped_kernel<T>, dim3((unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(256), 0, s, z, (T*)out, F, (size_t)n, limit, alpha);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_glu_clipped_f32(const float* z, void* out, int rows, int F, float limit, float alpha, cudaStream_t s) {
    return glu_clipped<float>(z, out, rows, F, limit, alpha, s);
}
extern "C" int bc_glu_clipped_bf16(const float* z, void* out, int rows, int F, float limit, float alpha, cudaStream_t s) {
    return glu_clipped<bf16>(z, out, rows, F, limit, alpha, s);
}

template <class T>
__global__ void gated_add_kernel(const T* h, const T* __restrict__ g, const float* y, float* x, int K, int E) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(h); PDL_FRESH(y); PDL_FRESH(x);
    const T* hr = h + (size_t)blockIdx.x * K;
    float s = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) s = fmaf(to_f32(hr[k]), to_f32(g[k]), s);
    s = block_sum(s, scratch);
    const float f = 1.0f / (1.0f + expf(-s));
    const float* yr = y + (size_t)blockIdx.x * E;
    float* xr = x + (size_t)blockIdx.x * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) xr[c] = fmaf(f, yr[c], xr[c]);
}
template <class T> static int gated_add(const void* h, const void* g, const float* y, float* x, int rows, int K, int E, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && K > 0 && E > 0, "gated_add: bad sizes rows=%d K=%d E=%d", rows, K, E);
    if (rows == 0) return BC_OK;
    bc_launch(gated_add_kernel<T>, dim3(rows), dim3(pick(K > E ? K : E)), 0, s, (const T*)h, (const T*)g, y, x, K, E);
    BC_LAUNCH_STATUS();
}
// h: [rows, K] and g: [K] of the activation type; y: [rows, E] float; x: [rows, E] float, changed in place.
extern "C" int bc_gated_add_f32(const void* h, const void* g, const float* y, float* x, int rows, int K, int E, cudaStream_t s) {
    return gated_add<float>(h, g, y, x, rows, K, E, s);
}
extern "C" int bc_gated_add_bf16(const void* h, const void* g, const float* y, float* x, int rows, int K, int E, cudaStream_t s) {
    return gated_add<bf16>(h, g, y, x, rows, K, E, s);
}

__global__ void table_route_kernel(const int* __restrict__ table, const int* __restrict__ tokens, const int* __restrict__ row_slot, int* __restrict__ choice,
                                   float* __restrict__ weight, int rows, int V, int E, int top) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * top) return;
    const int r = i / top, tok = tokens[r];
    int e = -1;
    if ((row_slot == nullptr || row_slot[r] >= 0) && tok >= 0 && tok < V) e = table[(size_t)tok * top + i % top];
    choice[i] = e >= 0 && e < E ? e : -1;
    weight[i] = 1.0f / (float)top;
}
// table: [V, top] int; tokens, row_slot: [rows] int (a negative slot: a padding row, which chooses nothing); choice: [rows, top] int; weight: the same, float.
extern "C" int bc_moe_table_route(const int* table, const int* tokens, const int* row_slot, int* choice, float* weight, int rows, int V, int E, int top,
                                  cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && V > 0 && E > 0 && top > 0 && top <= E, "moe_table_route: bad sizes rows=%d V=%d E=%d top=%d", rows, V, E, top);
    if (rows == 0) return BC_OK;
    bc_launch(table_route_kernel, dim3((rows * top + 127) / 128), dim3(128), 0, s, table, tokens, row_slot, choice, weight, rows, V, E, top);
    BC_LAUNCH_STATUS();
}
