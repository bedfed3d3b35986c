// Token embedding plus a hashed bigram embedding:
//   x[t] = E[id_t] + B[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]
// and, for the first token of a sequence (position 0), row `buckets` of B (the
// table has buckets + 1 rows).  The token before the first row of an entry is
// not in the step: it is the request's state, one int32 per request slot.  The
// block of an entry's first row reads it and then stores the entry's last
// token there for the next step; no other block touches that slot.
// The sum is made in 32-bit and written to the float32 residual stream and,
// when `out_act` is given, also rounded to the activation dtype.
#include "common.cuh"

using namespace ib;

template <typename TW>
__global__ void embed_hashed_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                    const int* __restrict__ row_entry, const int* __restrict__ cu_rows,
                                    const int* __restrict__ slot_ids, int* __restrict__ prev_state,
                                    int n_slots, const TW* __restrict__ table, const TW* __restrict__ bigram,
                                    float* __restrict__ out, bf16* __restrict__ out_act, int H, int V,
                                    long long buckets, long long mul_prev, long long mul_cur,
                                    unsigned* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ int s_prev;
    const int row = blockIdx.x;
    const int id = ids[row];
    if (threadIdx.x == 0) {
        const int e = row_entry[row];
        const int first = cu_rows[e];
        int prev = -1;  // -1: no token before this one
        if (row != first) {
            prev = ids[row - 1];
        } else {
            const int slot = slot_ids[e];
            if (slot >= 0 && slot < n_slots) {
                prev = prev_state[slot];
                prev_state[slot] = ids[cu_rows[e + 1] - 1];
            }
        }
        if (positions[row] == 0) prev = -1;
        s_prev = prev;
    }
    __syncthreads();
    const int prev = s_prev;
    float* o = out + (size_t)row * H;
    bf16* oa = out_act ? out_act + (size_t)row * H : nullptr;
    if (id < 0 || id >= V || prev >= V) {
        if (threadIdx.x == 0) atomicOr(err, IB_FLAG_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            o[i] = 0.f;
            if (oa) oa[i] = from_f32<bf16>(0.f);
        }
        return;
    }
    const long long b = prev < 0 ? buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    const TW* src = table + (size_t)id * H;
    const TW* bsrc = bigram + (size_t)b * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(src[i]) + to_f32(bsrc[i]);
        o[i] = v;
        if (oa) oa[i] = from_f32<bf16>(v);
    }
}

IB_EXPORT int ib_embed_hashed(const int* ids, const int* positions, const int* row_entry, const int* cu_rows,
                              const int* slot_ids, int* prev_state, int n_slots, const void* table,
                              const void* bigram, int table_dtype, float* out, void* out_act, int n_rows, int H,
                              int V, long long buckets, long long mul_prev, long long mul_cur, unsigned* err,
                              void* stream) {
    if (n_rows <= 0) return IB_OK;
    if (H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0 || n_slots <= 0 || !ids || !positions ||
        !row_entry || !cu_rows || !slot_ids || !prev_state || !table || !bigram || !out || !err)
        return IB_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    cudaError_t le;
    if (table_dtype == 0)
        le = launch_kernel(embed_hashed_kernel<float>, dim3(n_rows), dim3(threads), 0, s, ids, positions, row_entry,
                           cu_rows, slot_ids, prev_state, n_slots, (const float*)table, (const float*)bigram, out,
                           (bf16*)out_act, H, V, buckets, mul_prev, mul_cur, err);
    else if (table_dtype == 1)
        le = launch_kernel(embed_hashed_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, ids, positions, row_entry,
                           cu_rows, slot_ids, prev_state, n_slots, (const bf16*)table, (const bf16*)bigram, out,
                           (bf16*)out_act, H, V, buckets, mul_prev, mul_cur, err);
    else
        return IB_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
