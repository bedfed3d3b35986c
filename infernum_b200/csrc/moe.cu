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
