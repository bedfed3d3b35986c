// Token-by-token scans of recurrent mixers whose per-head state is a matrix of
// ROWS x P 32-bit floats (ROWS = IB_ROWS, fixed when this file is compiled; P at
// run time).  The state lives in the request's state slot and is carried from
// step to step; inside a step the tokens of an entry are walked in order, so a
// position's result is the same however the prompt was cut.
//
//   wkv:  o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])        (u only for the current token)
//         S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j],   w_t[i] = exp(-exp(z_t[i] + w0[i]))
//   ssd:  S[n][p] <- exp(-exp(A_log) dt_t) S[n][p] + dt_t B_t[n] x_t[p],  dt_t = softplus(dt_raw + dt_bias)
//         y_t[p] = sum_n C_t[n] S[n][p] + D x_t[p]
//
// One CTA per (entry, head, slice of columns).  A column j of the state is held
// by SPLIT neighbouring lanes, each with ROWS / SPLIT rows in registers (row
// i = ii * SPLIT + part); a token's per-row factors are staged in shared memory
// for CHUNK tokens at a time, one vector load per row; the partial sums of the
// SPLIT lanes meet by shuffles in a fixed order.  Decays, step sizes and the
// state are 32-bit; r, k, v, x, B, C arrive in the activation dtype.
#include "common.cuh"

using namespace ib;

#ifndef IB_ROWS
#error "compile with -DIB_ROWS=<rows of the state matrix>"
#endif

constexpr int ROWS = IB_ROWS;
constexpr int SPLIT = (ROWS % 8 == 0 && ROWS >= 128) ? 8 : (ROWS % 4 == 0 ? 4 : (ROWS % 2 == 0 ? 2 : 1));
constexpr int RPT = ROWS / SPLIT;  // rows of a column one thread holds
constexpr int CHUNK = ROWS <= 128 ? 16 : (ROWS <= 256 ? 8 : 4);
static_assert(ROWS >= 1 && ROWS <= 512, "state rows out of range");

__device__ __forceinline__ float split_sum(float v) {
#pragma unroll
    for (int o = 1; o < SPLIT; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct WkvParams {
    const void* r;
    const void* k;
    const void* v;
    int ld;             // row stride of r, k, v (elements)
    const float* z;     // decay pre-activation [rows][heads * ROWS]
    const float* w0;    // [heads * ROWS]
    const float* u;     // [heads * ROWS]
    float* state;       // request slot s, head h: state + s * state_stride + h * ROWS * P
    long long state_stride;
    const int* cu_rows;
    const int* slot_ids;
    float* out;         // [rows][heads * P]
    int heads, P, cols; // cols: columns of one CTA
};

template <typename T>
__global__ void __launch_bounds__(512) wkv_scan_kernel(const WkvParams p) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 smem4[];
    float4* s_f = smem4;                                         // [CHUNK][ROWS]: r, k, w, u * k
    float* s_v = reinterpret_cast<float*>(smem4 + CHUNK * ROWS);  // [CHUNK][cols]
    const int e = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * p.cols;
    const int first = p.cu_rows[e], end = p.cu_rows[e + 1];
    if (end <= first) return;
    const int part = threadIdx.x % SPLIT;
    const int col_raw = threadIdx.x / SPLIT;
    const bool active = col_raw < p.cols;
    const int col = active ? col_raw : p.cols - 1;
    float* st = p.state + (long long)p.slot_ids[e] * p.state_stride + (size_t)head * ROWS * p.P;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = st[(size_t)(ii * SPLIT + part) * p.P + j0 + col];
    const T* r = (const T*)p.r;
    const T* k = (const T*)p.k;
    const T* v = (const T*)p.v;
    const size_t hk = (size_t)head * ROWS, hp = (size_t)head * p.P;
    const int ldz = p.heads * ROWS, ldo = p.heads * p.P;

    for (int c0 = first; c0 < end; c0 += CHUNK) {
        const int nt = min(CHUNK, end - c0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * ROWS; idx += blockDim.x) {
            const int t = idx / ROWS, i = idx % ROWS;
            const size_t row = (size_t)(c0 + t);
            const float rr = to_f32(r[row * p.ld + hk + i]);
            const float kk = to_f32(k[row * p.ld + hk + i]);
            const float w = expf(-expf(p.z[row * ldz + hk + i] + p.w0[hk + i]));
            s_f[t * ROWS + i] = make_float4(rr, kk, w, p.u[hk + i] * kk);
        }
        for (int idx = threadIdx.x; idx < nt * p.cols; idx += blockDim.x) {
            const int t = idx / p.cols, jj = idx % p.cols;
            s_v[t * p.cols + jj] = to_f32(v[(size_t)(c0 + t) * p.ld + hp + j0 + jj]);
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vj = s_v[t * p.cols + col];
            const float4* f = s_f + t * ROWS + part;
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) {
                const float4 q = f[ii * SPLIT];
                acc = fmaf(q.x, fmaf(q.w, vj, S[ii]), acc);
                S[ii] = fmaf(q.z, S[ii], q.y * vj);
            }
            acc = split_sum(acc);
            if (active && part == 0) p.out[(size_t)(c0 + t) * ldo + hp + j0 + col] = acc;
        }
    }
    if (active) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) st[(size_t)(ii * SPLIT + part) * p.P + j0 + col] = S[ii];
    }
}

struct SsdParams {
    const void* xbc;   // conv output rows: [x: heads * P | B: groups * ROWS | C: groups * ROWS]
    int ld_xbc;
    const void* dt;    // raw step sizes, one per head, rows ld_dt apart
    int ld_dt;
    const float* dt_bias;
    const float* a_log;
    const float* d_skip;
    float* state;
    long long state_stride;
    const int* cu_rows;
    const int* slot_ids;
    float* out;        // [rows][heads * P]
    int heads, groups, P, cols;
};

template <typename T>
__global__ void __launch_bounds__(512) ssd_scan_kernel(const SsdParams p) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float4 smem4[];
    float2* s_bc = reinterpret_cast<float2*>(smem4);               // [CHUNK][ROWS]: dt * B, C
    float* s_x = reinterpret_cast<float*>(s_bc + CHUNK * ROWS);     // [CHUNK][cols]
    float* s_dt = s_x + CHUNK * p.cols;                             // [CHUNK]
    float* s_da = s_dt + CHUNK;                                     // [CHUNK]
    const int e = blockIdx.x, head = blockIdx.y, j0 = blockIdx.z * p.cols;
    const int first = p.cu_rows[e], end = p.cu_rows[e + 1];
    if (end <= first) return;
    const int part = threadIdx.x % SPLIT;
    const int col_raw = threadIdx.x / SPLIT;
    const bool active = col_raw < p.cols;
    const int col = active ? col_raw : p.cols - 1;
    float* st = p.state + (long long)p.slot_ids[e] * p.state_stride + (size_t)head * ROWS * p.P;
    float S[RPT];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) S[ii] = st[(size_t)(ii * SPLIT + part) * p.P + j0 + col];
    const T* xbc = (const T*)p.xbc;
    const T* dtp = (const T*)p.dt;
    const int inner = p.heads * p.P;
    const int grp = head / (p.heads / p.groups);
    const size_t b_off = (size_t)inner + (size_t)grp * ROWS;
    const size_t c_off = b_off + (size_t)p.groups * ROWS;
    const float a_neg = -expf(p.a_log[head]);
    const float bias = p.dt_bias[head], dsk = p.d_skip[head];

    for (int c0 = first; c0 < end; c0 += CHUNK) {
        const int nt = min(CHUNK, end - c0);
        __syncthreads();
        if (threadIdx.x < nt) {
            const float raw = to_f32(dtp[(size_t)(c0 + threadIdx.x) * p.ld_dt + head]) + bias;
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            s_dt[threadIdx.x] = dt;
            s_da[threadIdx.x] = expf(a_neg * dt);
        }
        for (int idx = threadIdx.x; idx < nt * p.cols; idx += blockDim.x) {
            const int t = idx / p.cols, jj = idx % p.cols;
            s_x[t * p.cols + jj] = to_f32(xbc[(size_t)(c0 + t) * p.ld_xbc + (size_t)head * p.P + j0 + jj]);
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * ROWS; idx += blockDim.x) {
            const int t = idx / ROWS, n = idx % ROWS;
            const size_t row = (size_t)(c0 + t) * p.ld_xbc;
            s_bc[t * ROWS + n] = make_float2(s_dt[t] * to_f32(xbc[row + b_off + n]), to_f32(xbc[row + c_off + n]));
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float xj = s_x[t * p.cols + col];
            const float da = s_da[t];
            const float2* f = s_bc + t * ROWS + part;
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < RPT; ++ii) {
                const float2 q = f[ii * SPLIT];
                S[ii] = fmaf(da, S[ii], q.x * xj);
                acc = fmaf(q.y, S[ii], acc);
            }
            acc = split_sum(acc);
            if (active && part == 0)
                p.out[(size_t)(c0 + t) * inner + (size_t)head * p.P + j0 + col] = fmaf(dsk, xj, acc);
        }
    }
    if (active) {
#pragma unroll
        for (int ii = 0; ii < RPT; ++ii) st[(size_t)(ii * SPLIT + part) * p.P + j0 + col] = S[ii];
    }
}

IB_EXPORT int ib_scan_rows() { return ROWS; }
IB_EXPORT int ib_scan_split() { return SPLIT; }

static int scan_geometry(int P, int col_slices, int* cols, int* threads) {
    if (P <= 0 || col_slices <= 0 || P % col_slices) return IB_ERR_BAD_ARG;
    *cols = P / col_slices;
    *threads = ((*cols * SPLIT + 31) / 32) * 32;
    if (*threads > 512) return IB_ERR_TOO_LARGE;
    return IB_OK;
}

// r, k, v: [rows][heads * ROWS] (v: heads * P) with row stride `ld`; z float32
// [rows][heads * ROWS]; out float32 [rows][heads * P].  `col_slices` CTAs share the
// columns of a head (it must divide P).
IB_EXPORT int ib_wkv_scan(const void* r, const void* k, const void* v, int ld, int act_dtype, const float* z,
                          const float* w0, const float* u, float* state, long long state_stride,
                          const int* cu_rows, const int* slot_ids, float* out, int n_entries, int heads, int P,
                          int col_slices, void* stream) {
    if (n_entries <= 0) return IB_OK;
    if (!r || !k || !v || !z || !w0 || !u || !state || !cu_rows || !slot_ids || !out || heads <= 0) return IB_ERR_BAD_ARG;
    int cols, threads;
    const int g = scan_geometry(P, col_slices, &cols, &threads);
    if (g != IB_OK) return g;
    WkvParams p{r, k, v, ld, z, w0, u, state, state_stride, cu_rows, slot_ids, out, heads, P, cols};
    const size_t smem = (size_t)CHUNK * ROWS * sizeof(float4) + (size_t)CHUNK * cols * sizeof(float);
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    dim3 grid(n_entries, heads, col_slices);
    cudaError_t le;
    if (act_dtype == 0) le = launch_kernel(wkv_scan_kernel<float>, grid, dim3(threads), smem, (cudaStream_t)stream, p);
    else if (act_dtype == 1) le = launch_kernel(wkv_scan_kernel<bf16>, grid, dim3(threads), smem, (cudaStream_t)stream, p);
    else return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}

IB_EXPORT int ib_ssd_scan(const void* xbc, int ld_xbc, const void* dt, int ld_dt, int act_dtype,
                          const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                          long long state_stride, const int* cu_rows, const int* slot_ids, float* out,
                          int n_entries, int heads, int groups, int P, int col_slices, void* stream) {
    if (n_entries <= 0) return IB_OK;
    if (!xbc || !dt || !dt_bias || !a_log || !d_skip || !state || !cu_rows || !slot_ids || !out || heads <= 0 ||
        groups <= 0 || heads % groups)
        return IB_ERR_BAD_ARG;
    int cols, threads;
    const int g = scan_geometry(P, col_slices, &cols, &threads);
    if (g != IB_OK) return g;
    SsdParams p{xbc, ld_xbc, dt, ld_dt, dt_bias, a_log, d_skip, state, state_stride, cu_rows, slot_ids, out,
                heads, groups, P, cols};
    const size_t smem = (size_t)CHUNK * ROWS * sizeof(float2) + (size_t)CHUNK * (cols + 2) * sizeof(float);
    if (smem > 48 * 1024) return IB_ERR_TOO_LARGE;
    dim3 grid(n_entries, heads, col_slices);
    cudaError_t le;
    if (act_dtype == 0) le = launch_kernel(ssd_scan_kernel<float>, grid, dim3(threads), smem, (cudaStream_t)stream, p);
    else if (act_dtype == 1) le = launch_kernel(ssd_scan_kernel<bf16>, grid, dim3(threads), smem, (cudaStream_t)stream, p);
    else return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
