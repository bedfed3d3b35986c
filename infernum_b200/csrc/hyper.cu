// Several residual streams per token (hyper-connections), a token embedding with
// an additive sinusoidal position vector, and a scale on the logits.
//
// Streams.  A token carries S copies x_0 .. x_{S-1} of the residual, stored side
// by side in 32-bit: x[row][s][H].  A sub-layer q reads one mixture of them and
// writes its result y back into all of them:
//   read   u      = sum_s a[s] x_s                      (a: `read`, null = all ones)
//   write  x_t'   = sum_s M[s][t] x_s + c[t] y          (M: `mix` [from][to], c: `out_coef`)
// `hc_norm_kernel` does the write of the sub-layer before (optional), the read of
// the next one and its norm in one pass over the row:
//   y_norm = (u - mean(u)) * rsqrt(var(u) + eps) * w (+ b)      (centred)
//   y_norm =  u            * rsqrt(mean(u^2) + eps) * w (+ b)   (otherwise)
// With `row_idx` only those rows are read and nothing is written back (the final
// norm on the rows whose logits are wanted).  Everything is 32-bit; the sums over
// the streams run in the order s = 0 .. S-1.
#include "common.cuh"

using namespace ib;

#define IB_MAX_STREAMS 8

__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const unsigned*>(&a);
    t.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}

// W = 4: four neighbouring columns a thread (H a multiple of 4, 16-byte loads of the streams);
// W = 1: any H.  The arithmetic per column and the order of the sums over the streams are the same.
template <typename TD, typename TW, typename TO, int W>
__global__ void hc_norm_kernel(float* __restrict__ x, const TD* __restrict__ y, const float* __restrict__ mix,
                               const float* __restrict__ out_coef, const float* __restrict__ read,
                               const TW* __restrict__ weight, const TW* __restrict__ bias, TO* __restrict__ out,
                               const int* __restrict__ row_idx, int S, int H, float eps, int centred,
                               int write_back) {
    pdl_trigger();
    extern __shared__ float4 hc_row4[];
    float* hc_row = reinterpret_cast<float*>(hc_row4);
    __shared__ float scratch[33];
    __shared__ float s_mix[IB_MAX_STREAMS * IB_MAX_STREAMS], s_out[IB_MAX_STREAMS], s_read[IB_MAX_STREAMS];
    // (the coefficients are weights: no kernel writes them, so they may be read before the wait)
    if (threadIdx.x < S * S) s_mix[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = out_coef ? out_coef[threadIdx.x] : 0.f;
        s_read[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
    }
    pdl_wait();
    __syncthreads();
    const int row = blockIdx.x;
    const int src = row_idx ? row_idx[row] : row;
    float* xr = x + (size_t)src * S * H;
    const TD* yr = y ? y + (size_t)src * H : nullptr;

    float sum = 0.f;
    for (int i = threadIdx.x * W; i < H; i += blockDim.x * W) {
        float old[IB_MAX_STREAMS][W];
#pragma unroll
        for (int s = 0; s < IB_MAX_STREAMS; ++s) {
            if (s < S) {
                if (W == 4) load4(xr + (size_t)s * H + i, reinterpret_cast<float(&)[4]>(old[s]));
                else old[s][0] = xr[(size_t)s * H + i];
            }
        }
        float u[W];
#pragma unroll
        for (int k = 0; k < W; ++k) u[k] = 0.f;
        if (yr) {
            float yv[W];
            if (W == 4) load4(yr + i, reinterpret_cast<float(&)[4]>(yv));
            else yv[0] = to_f32(yr[i]);
#pragma unroll
            for (int t = 0; t < IB_MAX_STREAMS; ++t) {
                if (t >= S) break;
                float nv[W];
#pragma unroll
                for (int k = 0; k < W; ++k) nv[k] = 0.f;
#pragma unroll
                for (int s = 0; s < IB_MAX_STREAMS; ++s) {
                    if (s < S) {
#pragma unroll
                        for (int k = 0; k < W; ++k) nv[k] += s_mix[s * S + t] * old[s][k];
                    }
                }
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    nv[k] += s_out[t] * yv[k];
                    u[k] += s_read[t] * nv[k];
                }
                if (write_back) {
                    if (W == 4) store4(xr + (size_t)t * H + i, reinterpret_cast<const float(&)[4]>(nv));
                    else xr[(size_t)t * H + i] = nv[0];
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < IB_MAX_STREAMS; ++s) {
                if (s < S) {
#pragma unroll
                    for (int k = 0; k < W; ++k) u[k] += s_read[s] * old[s][k];
                }
            }
        }
#pragma unroll
        for (int k = 0; k < W; ++k) {
            hc_row[i + k] = u[k];
            sum += u[k];
        }
    }
    if (!out) return;
    float mean = 0.f;
    if (centred) mean = block_sum(sum, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x * W; i < H; i += blockDim.x * W) {
#pragma unroll
        for (int k = 0; k < W; ++k) {
            const float c = hc_row[i + k] - mean;
            ss += c * c;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x * W; i < H; i += blockDim.x * W) {
        float wv[W], bv[W], v[W];
        if (W == 4) {
            load4(weight + i, reinterpret_cast<float(&)[4]>(wv));
            if (bias) load4(bias + i, reinterpret_cast<float(&)[4]>(bv));
        } else {
            wv[0] = to_f32(weight[i]);
            if (bias) bv[0] = to_f32(bias[i]);
        }
#pragma unroll
        for (int k = 0; k < W; ++k) {
            v[k] = (hc_row[i + k] - mean) * inv * wv[k];
            if (bias) v[k] += bv[k];
        }
        if (W == 4) store4(out + (size_t)row * H + i, reinterpret_cast<const float(&)[4]>(v));
        else out[(size_t)row * H + i] = from_f32<TO>(v[0]);
    }
}

template <typename TD, typename TW, typename TO>
static int launch_hc(float* x, const void* y, const float* mix, const float* out_coef, const float* read,
                     const void* weight, const void* bias, void* out, const int* row_idx, int n_rows, int S, int H,
                     float eps, int centred, int write_back, cudaStream_t s) {
    const bool vec = H % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)y & 15) && !((uintptr_t)out & 15) &&
                     !((uintptr_t)weight & 15) && !((uintptr_t)bias & 15);
    const int items = vec ? H / 4 : H;
    int threads = 128;
    if (items >= 4096) threads = 1024;
    else if (items >= 1024) threads = 512;
    else if (items >= 512) threads = 256;
    const size_t smem = (size_t)H * sizeof(float) + 16;
    auto kernel = vec ? hc_norm_kernel<TD, TW, TO, 4> : hc_norm_kernel<TD, TW, TO, 1>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return IB_ERR_TOO_LARGE;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaError_t le = launch_kernel(kernel, dim3(n_rows), dim3(threads), smem, s, x, (const TD*)y, mix, out_coef,
                                   read, (const TW*)weight, (const TW*)bias, (TO*)out, row_idx, S, H, eps, centred,
                                   write_back);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// x [rows][S][H] float32.  y (null: no write) is in the activation dtype, as is
// `out` (null: only the write is done); mix [S][S], out_coef [S], read [S] are
// float32 (read null: ones); weight and bias share `weight_dtype`.
IB_EXPORT int ib_hc_norm(float* x, const void* y, const float* mix, const float* out_coef, const float* read,
                         const void* weight, const void* bias, int weight_dtype, void* out, int act_dtype,
                         const int* row_idx, int n_rows, int S, int H, float eps, int centred, void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (!x || H <= 0 || S <= 0 || S > IB_MAX_STREAMS) return IB_ERR_BAD_ARG;
    if (y && (!mix || !out_coef)) return IB_ERR_BAD_ARG;
    if (out && (!weight || !(eps > 0.f))) return IB_ERR_BAD_ARG;
    if (!out && !y) return IB_OK;
    const int write_back = row_idx ? 0 : 1;
    cudaStream_t s = (cudaStream_t)stream;
    const int key = act_dtype * 10 + weight_dtype;
    switch (key) {
        case 0: return launch_hc<float, float, float>(x, y, mix, out_coef, read, weight, bias, out, row_idx, n_rows, S, H, eps, centred, write_back, s);
        case 1: return launch_hc<float, bf16, float>(x, y, mix, out_coef, read, weight, bias, out, row_idx, n_rows, S, H, eps, centred, write_back, s);
        case 10: return launch_hc<bf16, float, bf16>(x, y, mix, out_coef, read, weight, bias, out, row_idx, n_rows, S, H, eps, centred, write_back, s);
        case 11: return launch_hc<bf16, bf16, bf16>(x, y, mix, out_coef, read, weight, bias, out, row_idx, n_rows, S, H, eps, centred, write_back, s);
        default: return IB_ERR_UNSUPPORTED;
    }
}

// ---------------------------------------------------------------------------
// Embedding with an additive sinusoidal position vector, written to S streams:
//   out[t][s][c] = table[id_t][c] + (c even ? sin : cos)(p_t * inv_freq[c / 2])
// The angle is the 32-bit product of the position and a float32 frequency.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_sinusoid_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                      const TW* __restrict__ table, const float* __restrict__ inv_freq,
                                      float* __restrict__ out, int H, int V, int S, unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    const float p = (float)positions[row];
    float* o = out + (size_t)row * S * H;
    const bool bad = id < 0 || id >= V;
    if (bad && threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_TOKEN);
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.f;
        if (!bad) {
            const float a = p * inv_freq[i >> 1];
            v = to_f32(src[i]) + ((i & 1) ? cosf(a) : sinf(a));
        }
        for (int s = 0; s < S; ++s) o[(size_t)s * H + i] = v;
    }
}

IB_EXPORT int ib_embed_sinusoid(const int* ids, const int* positions, const void* table, int table_dtype,
                                const float* inv_freq, float* out, int n_rows, int H, int V, int S, unsigned* err,
                                void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || V <= 0 || S <= 0 || !ids || !positions || !table || !inv_freq || !out || !err) return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t le;
    if (table_dtype == 0)
        le = launch_kernel(embed_sinusoid_kernel<float>, dim3(n_rows), dim3(threads), 0, s, ids, positions,
                           (const float*)table, inv_freq, out, H, V, S, err);
    else if (table_dtype == 1)
        le = launch_kernel(embed_sinusoid_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, ids, positions,
                           (const bf16*)table, inv_freq, out, H, V, S, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

// Logits times a constant, in place (32-bit).
__global__ void scale_inplace_kernel(float* __restrict__ x, size_t n, float scale) {
    pdl_trigger();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= scale;
}

IB_EXPORT int ib_scale_inplace(float* x, long long n, float scale, void* stream) {
    if (n <= 0) return IB_OK;
    if (!x) return IB_ERR_BAD_ARG;
    cudaError_t le = launch_kernel(scale_inplace_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                   (cudaStream_t)stream, x, (size_t)n, scale);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
