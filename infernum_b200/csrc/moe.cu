// Routing of a mixture of experts.
//   z = router logits [N, E] (32-bit) + bias;  the `top` largest are chosen (the
//   lower index among equals), and their weights are the softmax over the chosen
//   logits only.  Written two ways: the lists ids[N, top] / weights[N, top] in
//   order of falling logit, and the dense row gate[N, E] that holds a chosen
//   expert's weight and 0 elsewhere.
// One warp per row; the row is kept in shared memory and a chosen logit is
// struck out there.
#include "common.cuh"

using namespace ib;

// Router logits z[n, e] = sum_k x[n, k] w[e, k] in 32-bit: one warp per (row,
// expert), lanes stride over k, then a fixed tree over the lanes; a row's logits do
// not depend on the batch.  The product is skinny (a handful of experts, K in the
// thousands): a tiled product would leave one CTA walking all of K.
template <typename TX, typename TW>
__global__ void router_logits_kernel(const TX* __restrict__ x, int ldx, const TW* __restrict__ w, int ldw,
                                     float* __restrict__ z, int n_rows, int E, int K) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_rows * E) return;
    const int n = warp / E, e = warp % E;
    const TX* xr = x + (size_t)n * ldx;
    const TW* wr = w + (size_t)e * ldw;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(to_f32(xr[k]), to_f32(wr[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) z[(size_t)n * E + e] = acc;
}

IB_EXPORT int ib_router_logits(const void* x, int x_dtype, int ldx, const void* w, int w_dtype, int ldw, float* z,
                               int n_rows, int E, int K, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || !w || !z || E <= 0 || K <= 0 || ldx < K || ldw < K) return IB_ERR_BAD_ARG;
    const long long warps = (long long)n_rows * E;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t le;
    if (x_dtype == 0 && w_dtype == 0)
        le = launch_kernel(router_logits_kernel<float, float>, dim3(blocks), dim3(256), 0, s, (const float*)x, ldx,
                           (const float*)w, ldw, z, n_rows, E, K);
    else if (x_dtype == 1 && w_dtype == 1)
        le = launch_kernel(router_logits_kernel<bf16, bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)x, ldx,
                           (const bf16*)w, ldw, z, n_rows, E, K);
    else if (x_dtype == 1 && w_dtype == 0)
        le = launch_kernel(router_logits_kernel<bf16, float>, dim3(blocks), dim3(256), 0, s, (const bf16*)x, ldx,
                           (const float*)w, ldw, z, n_rows, E, K);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int E,
                                 int top, int* __restrict__ ids, float* __restrict__ weights,
                                 float* __restrict__ gate) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float z[];
    const int row = blockIdx.x, lane = threadIdx.x;
    const float* src = logits + (size_t)row * ld;
    for (int e = lane; e < E; e += 32) {
        z[e] = src[e] + (bias ? bias[e] : 0.f);
        if (gate) gate[(size_t)row * E + e] = 0.f;
    }
    __syncwarp();
    float zmax = 0.f, denom = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }   // (NaN never wins)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = k < E ? k : 0;  // a row of NaN: any expert, weight NaN
        if (k == 0) zmax = best;
        const float p = expf(best - zmax);
        denom += p;
        if (lane == 0) {
            ids[(size_t)row * top + k] = at;
            weights[(size_t)row * top + k] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            const float w = weights[(size_t)row * top + k] / denom;
            weights[(size_t)row * top + k] = w;
            if (gate) gate[(size_t)row * E + ids[(size_t)row * top + k]] = w;
        }
    }
}

IB_EXPORT int ib_moe_route(const float* logits, int ld, const float* bias, int E, int top, int* ids,
                           float* weights, float* gate, int n_rows, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!logits || !ids || !weights || E <= 0 || top <= 0 || top > E || ld < E) return IB_ERR_BAD_ARG;
    if ((size_t)E * sizeof(float) > 48 * 1024) return IB_ERR_TOO_LARGE;
    cudaError_t le = launch_kernel(moe_route_kernel, dim3(n_rows), dim3(32), (size_t)E * sizeof(float),
                                   (cudaStream_t)stream, logits, ld, bias, E, top, ids, weights, gate);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
