// Small kernels on the float residual stream and on scores.
//
//   softcap:  s <- cap * tanh(s / cap), in place, on float scores
//   scale:    s <- factor * s, in place, on float scores
//   add_bias: x[r] += b, on float rows (the bias of a product that adds into them)
//   reentry:  for a stretch of layers that runs several times: cat[r] = [x[r]; x0[r]] in the activation
//             type (the operand of the product that mixes the stream with the embedding's output) and
//             x[r] <- step (the vector of the pass), so that the product's epilogue adds onto it
#include "common.cuh"

__global__ void softcap_kernel(float* __restrict__ s, size_t n, float cap) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(s);
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) s[i] = cap * tanhf(s[i] * inv);
}

extern "C" int bc_softcap_f32(float* scores, long long n, float cap, cudaStream_t s) {
    BC_CHECK_ARG(n >= 0 && cap > 0.0f, "softcap: bad sizes n=%lld cap=%g", n, (double)cap);
    if (n == 0) return BC_OK;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    bc_launch(softcap_kernel, dim3((unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(threads), 0, s, scores, (size_t)n, cap);
    BC_LAUNCH_STATUS();
}

__global__ void scale_kernel(float* __restrict__ s, size_t n, float factor) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(s);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) s[i] *= factor;
}

extern "C" int bc_scale_f32(float* scores, long long n, float factor, cudaStream_t s) {
    BC_CHECK_ARG(n >= 0, "scale: bad size n=%lld", n);
    if (n == 0) return BC_OK;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    bc_launch(scale_kernel, dim3((unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(threads), 0, s, scores, (size_t)n, factor);
    BC_LAUNCH_STATUS();
}

__global__ void add_bias_kernel(float* __restrict__ x, const float* __restrict__ b, int E, size_t n) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(x);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += b[i % E];
}

// x: [rows, E] float; b: [E] float.
extern "C" int bc_add_bias_f32(float* x, const float* b, int rows, int E, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0, "add_bias: bad sizes rows=%d E=%d", rows, E);
    const long long n = (long long)rows * E;
    if (n == 0) return BC_OK;
    const long long blocks = (n + 255) / 256;
    bc_launch(add_bias_kernel, dim3((unsigned)(blocks < 65535 * 16 ? blocks : 65535 * 16)), dim3(256), 0, s, x, b, E, (size_t)n);
    BC_LAUNCH_STATUS();
}

template <class T>
__global__ void reentry_kernel(float* __restrict__ x, const float* __restrict__ x0, const float* __restrict__ step, T* __restrict__ cat, int E) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(x); PDL_FRESH(x0);
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * E;
    const float* x0r = x0 + (size_t)r * E;
    T* out = cat + (size_t)r * 2 * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        out[c] = from_f32<T>(xr[c]);
        out[E + c] = from_f32<T>(x0r[c]);
        xr[c] = step[c];
    }
}

template <class T>
static int reentry(float* x, const float* x0, const float* step, void* cat, int rows, int E, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0, "reentry: bad sizes rows=%d E=%d", rows, E);
    if (rows == 0) return BC_OK;
    bc_launch(reentry_kernel<T>, dim3(rows), dim3(E >= 1024 ? 256 : 128), 0, s, x, x0, step, (T*)cat, E);
    BC_LAUNCH_STATUS();
}
// x, x0: [rows, E] float; step: [E] float; cat: [rows, 2 E] of the activation type.
extern "C" int bc_reentry_f32(float* x, const float* x0, const float* step, void* cat, int rows, int E, cudaStream_t s) {
    return reentry<float>(x, x0, step, cat, rows, E, s);
}
extern "C" int bc_reentry_bf16(float* x, const float* x0, const float* step, void* cat, int rows, int E, cudaStream_t s) {
    return reentry<bf16>(x, x0, step, cat, rows, E, s);
}
