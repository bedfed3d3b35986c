// Norm of a scaled sum, for layers that norm after the residual add:
//   s = alpha * residual[src] (+ delta[src])
//   centred:   y = (s - mean(s)) * rsqrt(mean((s - mean(s))^2) + eps) * w (+ b)
//   otherwise: y =  s            * rsqrt(mean(s^2) + eps)             * w (+ b)
// `store` = 1 writes y back over residual[src] in 32-bit (the normed sum is the
// new residual stream); `out` (optional) receives y in the activation dtype,
// compact when `row_idx` selects rows.  One block per row; the row is held in
// shared memory, the mean is taken first and the variance from the deviations,
// everything in 32-bit, and the order of the additions depends on H and the
// block size only.
#include "common.cuh"

using namespace ib;

template <typename TD, typename TW, typename TO>
__global__ void scale_add_norm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                      const TW* __restrict__ weight, const TW* __restrict__ bias,
                                      TO* __restrict__ out, const int* __restrict__ row_idx, int H,
                                      float eps, float alpha, int centred, int store) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float ln_row[];
    __shared__ float scratch[33];
    const int row = blockIdx.x;
    const int src = row_idx ? row_idx[row] : row;
    float* r = residual + (size_t)src * H;
    const TD* d = delta ? delta + (size_t)src * H : nullptr;

    float sum = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = alpha * r[i];
        if (d) v += to_f32(d[i]);
        ln_row[i] = v;
        sum += v;
    }
    float mean = 0.f;
    if (centred) mean = block_sum(sum, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float c = ln_row[i] - mean;
        ss += c * c;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float y = (ln_row[i] - mean) * inv * to_f32(weight[i]);
        if (bias) y += to_f32(bias[i]);
        if (store) r[i] = y;
        if (out) out[(size_t)row * H + i] = from_f32<TO>(y);
    }
}

template <typename TD, typename TW, typename TO>
static int launch_norm(float* residual, const void* delta, const void* weight, const void* bias, void* out,
                       const int* row_idx, int n_rows, int H, float eps, float alpha, int centred, int store,
                       cudaStream_t s) {
    int threads = 256;
    if (H >= 8192) threads = 1024;
    else if (H >= 2048) threads = 512;
    else if (H <= 512) threads = 128;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return IB_ERR_TOO_LARGE;
        cudaError_t e = cudaFuncSetAttribute(scale_add_norm_kernel<TD, TW, TO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaError_t le = launch_kernel(scale_add_norm_kernel<TD, TW, TO>, dim3(n_rows), dim3(threads), smem, s,
                                   residual, (const TD*)delta, (const TW*)weight, (const TW*)bias, (TO*)out,
                                   row_idx, H, eps, alpha, centred, store);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// act_dtype is the type of `delta` and of `out` (0 = f32, 1 = bf16); weight and
// bias share `weight_dtype`.  `out`, `delta`, `bias` and `row_idx` may be null.
IB_EXPORT int ib_scale_add_norm(float* residual, const void* delta, const void* weight, const void* bias,
                                int weight_dtype, void* out, int act_dtype, const int* row_idx, int n_rows,
                                int H, float eps, float alpha, int centred, int store, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || !residual || !weight || !(eps > 0.f)) return IB_ERR_BAD_ARG;
    if (store && row_idx) return IB_ERR_BAD_ARG;  // the rows a gather leaves out would keep the old stream
    cudaStream_t s = (cudaStream_t)stream;
    const int key = act_dtype * 10 + weight_dtype;
    switch (key) {
        case 0: return launch_norm<float, float, float>(residual, delta, weight, bias, out, row_idx, n_rows, H, eps, alpha, centred, store, s);
        case 1: return launch_norm<float, bf16, float>(residual, delta, weight, bias, out, row_idx, n_rows, H, eps, alpha, centred, store, s);
        case 10: return launch_norm<bf16, float, bf16>(residual, delta, weight, bias, out, row_idx, n_rows, H, eps, alpha, centred, store, s);
        case 11: return launch_norm<bf16, bf16, bf16>(residual, delta, weight, bias, out, row_idx, n_rows, H, eps, alpha, centred, store, s);
        default: return IB_ERR_UNSUPPORTED;
    }
}

// Soft cap of logits in place: x <- cap * tanh(x / cap), 32-bit.
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

IB_EXPORT int ib_softcap(float* x, long long n, float cap, void* stream) {
    if (n <= 0) return IB_OK;
    if (!x || !(cap > 0.f)) return IB_ERR_BAD_ARG;
    cudaError_t le = launch_kernel(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                   (cudaStream_t)stream, x, (size_t)n, cap);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
