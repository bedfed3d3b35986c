// Attention of all heads over one cached latent per token, on the tensor cores
// (bf16 mma.sync m16n8k16, 32-bit accumulation, 32-bit softmax).
//
//   q_abs [N, H, W]      each head's query in latent space, then its rotated part
//   pool  [pages, 1, page_size, W]   each token's latent c (KV elements) followed
//                        by the rotated key part all heads share
//   out   [N, H, KV]     sum_j p_j c_j;  s_j = (q . pool_j) * scale over the
//                        visible keys max(0, p - window + 1) <= j <= p
//
// Every head reads the same keys, and a key's value is its own first KV
// elements.  So the rows of a step are packed with their heads on the M side
// of the MMA - packed row g = row * H + head - and a tile of keys fetched once
// serves all of them: S = Q K^T and O += P K[:, :KV] from the one tile in
// shared memory.  A CTA has RG groups of four warps; a group owns 16 * MT packed
// rows of one entry, all groups share the tile of keys.  Per tile of 32 keys each
// warp computes the scores of eight keys for its group's rows; the scores meet
// in shared memory, where the threads share out the rows for the softmax
// (running maximum and denominator per row, P rounded to bf16, all kept in
// shared memory); then each warp adds P V for its quarter of the KV value
// columns of its group's rows.
// Keys come by cp.async into two buffers, a row at a time through the block
// table; rows outside the request's keys or below every row's window are
// zero-filled, never read (their pages may belong to someone else by now).
// Key tiles start at absolute multiples of 32, so a row's result does not
// depend on how its prompt was cut.
//
// With `splits` > 1 the key tiles of a CTA's rows are shared out over
// gridDim.z CTAs that each write unnormalised sums, maxima and denominators
// to scratch; latent_combine_kernel merges them.  That is how a few decoded
// rows fill the machine.
//
// Built per (KV, W): -DLAT_KV=<kv_rank> -DLAT_W=<kv_rank + rot_dim>;
// KV a multiple of 32, W a multiple of 16.
#include "common.cuh"

using namespace ib;

#ifndef LAT_KV
#define LAT_KV 64
#endif
#ifndef LAT_W
#define LAT_W 96
#endif

namespace {
constexpr int KV = LAT_KV, W = LAT_W;
constexpr int KT = 32;            // keys per tile
constexpr int LDK = W + 8;        // row stride of Q and K tiles in shared memory (elements)
constexpr int LDS = KT + 1;       // row stride of the score tile (floats)
constexpr int NT = KV / 32;       // 8-column output tiles per warp
constexpr int KSTEPS = W / 16;
static_assert(KV % 32 == 0 && W % 16 == 0 && KV <= W, "latent attention: unsupported sizes");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A barrier of one group of four warps (ids 1, 2: id 0 is __syncthreads): the groups of a CTA
// meet only around the shared tile of keys and are free of each other in between.
__device__ __forceinline__ void group_sync(int group) {
    asm volatile("bar.sync %0, 128;\n" ::"r"(group + 1) : "memory");
}

struct LatentParams {
    const bf16* q; int q_rs, q_hs;
    const bf16* pool;
    bf16* out; int o_rs, o_hs;
    const int* cu_rows; const int* q_start; const int* tables; int max_blocks;
    int n_entries, heads, page_size, num_pages, window;
    float scale;
    int splits;
    float* part_o; float* part_ml;   // [splits, N * H, KV] and [splits, N * H, 2]
    int n_rows_total;
    unsigned* err;
};

constexpr int LDP = KT + 8;       // row stride of the P tile (bf16)

template <int MT, int RG>
__global__ void __launch_bounds__(128 * RG) latent_attention_kernel(const LatentParams p) {
    constexpr int M = 16 * MT * RG;
    constexpr int THREADS = 128 * RG;
    constexpr int TPR = THREADS / M;                              // threads that share a row's softmax (8 / MT)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [M][LDK]
    bf16* Ks = Qs + M * LDK;                                      // [2][KT][LDK]
    bf16* Ps = Ks + 2 * KT * LDK;                                 // [M][LDP]
    float* Ss = reinterpret_cast<float*>(Ps + M * LDP);           // [M][LDS]
    float* m_s = Ss + M * LDS;                                    // [M] running maximum
    float* l_s = m_s + M;                                         // [M] running denominator
    float* c_s = l_s + M;                                         // [M] this tile's correction of the sums so far
    int* slot_s = reinterpret_cast<int*>(c_s + M);                // [2][KT] where the key rows of a tile lie in the pool

    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.y;
    const int row0 = p.cu_rows[e], rows = p.cu_rows[e + 1] - row0;
    const int H = p.heads;
    const int g0 = blockIdx.x * M;                 // first packed row of this CTA
    if (g0 >= rows * H) return;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = (tid >> 5) & 3;               // which eight keys / which quarter of the value columns
    const int rbase = (tid >> 7) * 16 * MT;        // first row of this warp's group within the CTA's rows
    const int grp = lane >> 2, qd = lane & 3;
    const int pos0 = p.q_start[e];
    const int r_first = g0 / H;
    const int g_last = min(g0 + M, rows * H) - 1;
    const int r_last = g_last / H;
    // keys any row of the tile may see
    const int key_hi = pos0 + r_last;                                        // inclusive
    const int key_lo = p.window > 0 ? max(0, pos0 + r_first - p.window + 1) : 0;
    int t_lo = key_lo / KT, t_hi = key_hi / KT + 1;                           // key tiles [t_lo, t_hi)
    if (p.splits > 1) {
        const int per = (t_hi - t_lo + p.splits - 1) / p.splits;
        t_lo = t_lo + (int)blockIdx.z * per;
        t_hi = min(t_hi, t_lo + per);
    }
    const int* table = p.tables + (size_t)e * p.max_blocks;

    // ---- the queries of the tile into shared memory (rows beyond the entry: zero) ----
    constexpr int CH = W / 8;  // 16-byte pieces per row
    for (int it = tid; it < M * CH; it += THREADS) {
        const int m = it / CH, c = it % CH;
        const int g = g0 + m;
        bf16* dst = Qs + m * LDK + c * 8;
        if (g <= g_last) {
            const int r = g / H, h = g % H;
            cp_async16(dst, p.q + (size_t)(row0 + r) * p.q_rs + (size_t)h * p.q_hs + c * 8);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    // Where each key row of a tile lies in the pool is looked up once per tile (a thread a
    // row) and passed through shared memory: a look-up per 16-byte piece would put a
    // dependent load from the block table before every copy.
    auto load_keys = [&](int t, int buf) {
        if (tid < KT) {
            const int j = t * KT + tid;
            int slot = -1;   // the token's place in the pool, or -1: the row is zero-filled
            if (j >= key_lo && j <= key_hi) {
                const int blk = j / p.page_size;
                const int page = blk < p.max_blocks ? table[blk] : -1;
                if (page < 0 || page >= p.num_pages) atomicOr(p.err, IB_FLAG_BAD_PAGE);
                else slot = page * p.page_size + (j % p.page_size);
            }
            slot_s[buf * KT + tid] = slot;
        }
        __syncthreads();
        bf16* base = Ks + buf * KT * LDK;
        for (int it = tid; it < KT * CH; it += THREADS) {
            const int kr = it / CH, c = it % CH;
            bf16* dst = base + kr * LDK + c * 8;
            const int slot = slot_s[buf * KT + kr];
            if (slot >= 0)
                cp_async16(dst, p.pool + (size_t)slot * W + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    };
    if (t_lo < t_hi) load_keys(t_lo, 0);
    cp_async_commit();

    float o[MT][NT][4];
    int row_pos[MT][2];   // position of this thread's two rows per m-tile (-1: no such row)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int k = 0; k < 4; ++k) o[mt][nt][k] = 0.f;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int g = g0 + rbase + mt * 16 + grp + hf * 8;
            row_pos[mt][hf] = g <= g_last ? pos0 + g / H : -1;
        }
    }
    for (int i = tid; i < M; i += THREADS) {
        m_s[i] = -INFINITY;
        l_s[i] = 0.f;
    }

    for (int t = t_lo; t < t_hi; ++t) {
        const int buf = (t - t_lo) & 1;
        if (t + 1 < t_hi) load_keys(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* Kt = Ks + buf * KT * LDK;
        // ---- scores of this warp's eight keys for all rows -------------------------
        float s[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int k = 0; k < 4; ++k) s[mt][k] = 0.f;
#pragma unroll 4
        for (int ks = 0; ks < KSTEPS; ks += 2) {
            // B fragments of two k-steps at once (W / 16 may be odd: the last pair is cut)
            unsigned b[4];
            const bool two = ks + 1 < KSTEPS;
            {
                const int mat = lane >> 3;                       // 0,1: k-step ks; 2,3: k-step ks + 1
                int kcol = ks * 16 + mat * 8;
                if (!two && mat >= 2) kcol = ks * 16;            // (stays inside the row; unused)
                ldsm_x4(b, Kt + (warp * 8 + (lane & 7)) * LDK + kcol);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                unsigned a[4];
                ldsm_x4(a, Qs + (rbase + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + ks * 16 + (lane >> 4) * 8);
                mma16816(s[mt], a, b[0], b[1]);
                if (two) {
                    ldsm_x4(a, Qs + (rbase + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (ks + 1) * 16 + (lane >> 4) * 8);
                    mma16816(s[mt], a, b[2], b[3]);
                }
            }
        }
        // scale, mask, and into the shared score tile
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int hf = k >> 1;
                const int j = t * KT + warp * 8 + qd * 2 + (k & 1);
                const int rp = row_pos[mt][hf];
                const bool seen = rp >= 0 && j <= rp && (p.window <= 0 || j > rp - p.window);
                Ss[(rbase + mt * 16 + grp + hf * 8) * LDS + warp * 8 + qd * 2 + (k & 1)] = seen ? s[mt][k] * p.scale : -INFINITY;
            }
        group_sync(tid >> 7);   // (a group's threads take the softmax of the group's own rows)
        // ---- softmax: TPR threads a row; maximum, P (bf16) and denominator into shared memory ----
        {
            constexpr int KPT = KT / TPR;   // keys per thread
            const int row = tid / TPR, sub = tid % TPR;
            const float* srow = Ss + row * LDS + sub * KPT;
            float sv[KPT];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < KPT; ++j) {
                sv[j] = srow[j];
                mx = fmaxf(mx, sv[j]);
            }
#pragma unroll
            for (int o2 = TPR / 2; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
            const float m_old = m_s[row];
            mx = fmaxf(mx, m_old);
            const float base = mx == -INFINITY ? 0.f : mx;
            float sum = 0.f;
            bf16* prow = Ps + row * LDP + sub * KPT;
#pragma unroll
            for (int j = 0; j < KPT; j += 2) {
                const float p0 = __expf(sv[j] - base), p1 = __expf(sv[j + 1] - base);
                sum += p0 + p1;
                *reinterpret_cast<__nv_bfloat162*>(prow + j) = __floats2bfloat162_rn(p0, p1);
            }
#pragma unroll
            for (int o2 = TPR / 2; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
            if (sub == 0) {
                const float corr = __expf(m_old - base);    // exp(-inf) = 0 before the first seen key
                c_s[row] = corr;
                l_s[row] = l_s[row] * corr + sum;
                m_s[row] = mx;
            }
        }
        group_sync(tid >> 7);
        // ---- O += P V for this warp's rows and value columns ---------------------------
        {
            unsigned pa[MT][2][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float c0 = c_s[rbase + mt * 16 + grp], c1 = c_s[rbase + mt * 16 + grp + 8];
#pragma unroll
                for (int kk = 0; kk < 2; ++kk)
                    ldsm_x4(pa[mt][kk], Ps + (rbase + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[mt][nt][0] *= c0;
                    o[mt][nt][1] *= c0;
                    o[mt][nt][2] *= c1;
                    o[mt][nt][3] *= c1;
                }
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int nt = 0; nt < NT; nt += 2) {
                    unsigned v[4];
                    const int mat = lane >> 3;   // 0: keys 0-7 of n-tile nt, 1: keys 8-15, 2, 3: the same of n-tile nt + 1
                    int col = warp * (KV / 4) + (nt + (mat >> 1)) * 8;
                    if (nt + 1 >= NT && mat >= 2) col = warp * (KV / 4) + nt * 8;
                    ldsm_x4_trans(v, Kt + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * LDK + col);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma16816(o[mt][nt], pa[mt][kk], v[0], v[1]);
                        if (nt + 1 < NT) mma16816(o[mt][nt + 1], pa[mt][kk], v[2], v[3]);
                    }
                }
            }
        }
        __syncthreads();   // the key buffer and the score tile are free again
    }
    cp_async_wait<0>();
    __syncthreads();   // (with no key tile at all the rows' statistics were only just initialised)

    // ---- results ------------------------------------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int lr = rbase + mt * 16 + grp + hf * 8;
            const float l = l_s[lr];
            const int g = g0 + lr;
            if (g > g_last) continue;
            const int r = g / H, h = g % H;
            if (p.splits <= 1) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* dst = p.out + (size_t)(row0 + r) * p.o_rs + (size_t)h * p.o_hs + warp * (KV / 4) + qd * 2;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                        __floats2bfloat162_rn(o[mt][nt][hf * 2] * inv, o[mt][nt][hf * 2 + 1] * inv);
            } else {
                const size_t pr = (size_t)blockIdx.z * p.n_rows_total * H + (size_t)(row0 + r) * H + h;
                float* dst = p.part_o + pr * KV + warp * (KV / 4) + qd * 2;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[mt][nt][hf * 2], o[mt][nt][hf * 2 + 1]);
                if (warp == 0 && qd == 0) {
                    p.part_ml[pr * 2] = m_s[lr];
                    p.part_ml[pr * 2 + 1] = l;
                }
            }
        }
}

// out[row, head, :] = sum_s exp(m_s - M) O_s / sum_s exp(m_s - M) l_s over the splits.
// One block per (row, head): the splits' maxima and denominators are fetched side by side
// (a thread each), turned into one weight per split in shared memory, and every thread then
// sums its columns over the splits in split order, the loads of a column independent of each
// other.
__global__ void latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, int o_rs, int o_hs, int n_rows, int heads,
                                      int splits) {
    pdl_trigger();
    pdl_wait();
    __shared__ float w_s[64];     // splits <= 64
    __shared__ float m_sh[64], l_sh[64];
    const int pr = blockIdx.x;   // row * heads + head
    const int r = pr / heads, h = pr % heads;
    const size_t stride = (size_t)n_rows * heads;
    const int tid = threadIdx.x;
    if (tid < splits) {
        m_sh[tid] = part_ml[((size_t)tid * stride + pr) * 2];
        l_sh[tid] = part_ml[((size_t)tid * stride + pr) * 2 + 1];
    }
    __syncthreads();
    if (tid == 0) {
        float mx = -INFINITY;
        for (int s = 0; s < splits; ++s) mx = fmaxf(mx, m_sh[s]);
        float denom = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float w = m_sh[s] > -INFINITY ? __expf(m_sh[s] - mx) : 0.f;
            w_s[s] = w;
            denom += w * l_sh[s];
        }
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
        for (int s = 0; s < splits; ++s) w_s[s] *= inv;
    }
    __syncthreads();
    // four columns a thread, 16 bytes a load (KV is a multiple of 32, the scratch 16-byte aligned)
    for (int c = tid * 4; c < KV; c += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* src = part_o + (size_t)pr * KV + c;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(src + (size_t)s * stride * KV);
            const float w = w_s[s];
            acc.x += w * v.x;
            acc.y += w * v.y;
            acc.z += w * v.z;
            acc.w += w * v.w;
        }
        bf16* dst = out + (size_t)r * o_rs + (size_t)h * o_hs + c;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x, acc.y);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z, acc.w);
    }
}

template <int MT, int RG>
int launch_latent(const LatentParams& p, int max_packed_rows, cudaStream_t s) {
    constexpr int M = 16 * MT * RG;
    const size_t smem = (size_t)(M * LDK + 2 * KT * LDK + M * LDP) * sizeof(bf16) +
                        (size_t)(M * LDS + 3 * M) * sizeof(float) + (size_t)2 * KT * sizeof(int);
    static bool set = false;
    if (!set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<MT, RG>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const int tiles_x = (max_packed_rows + M - 1) / M;
    cudaError_t le = launch_kernel(latent_attention_kernel<MT, RG>, dim3(tiles_x, p.n_entries, p.splits),
                                   dim3(128 * RG), smem, s, p);
    if (le != cudaSuccess) return (int)le;
    IB_LAUNCH_CHECK();
    return IB_OK;
}
}  // namespace

IB_EXPORT int ib_attention_latent_kv() { return KV; }
IB_EXPORT int ib_attention_latent_width() { return W; }

IB_EXPORT long long ib_attention_latent_scratch_bytes(int n_rows, int heads, int splits) {
    return splits > 1 ? (long long)splits * n_rows * heads * (KV + 2) * (long long)sizeof(float) : 0;
}

// q [N, H, W] with row / head strides q_rs / q_hs (elements), out [N, H, KV] likewise; bf16.
// `mt`: 1, 2: that many sixteens of packed rows for four warps; 3: 32 rows, 4: 64 rows, for eight
// warps in two groups.
// `splits` > 1 needs scratch of
// ib_attention_latent_scratch_bytes.
IB_EXPORT int ib_attention_latent(const void* q, int q_rs, int q_hs, const void* pool, void* out, int o_rs, int o_hs,
                                  const int* cu_rows, const int* q_start, const int* tables, int max_blocks,
                                  int n_entries, int n_rows, int max_rows_per_entry, int heads, int page_size,
                                  int num_pages, int window, float scale, int mt, int splits, void* scratch,
                                  long long scratch_bytes, unsigned* err, void* stream) {
    if (n_entries <= 0 || n_rows <= 0) return IB_OK;
    if (!q || !pool || !out || !cu_rows || !q_start || !tables || !err || heads <= 0 || page_size <= 0 ||
        num_pages <= 0 || max_blocks <= 0 || max_rows_per_entry <= 0 || splits < 1 || splits > 64)
        return IB_ERR_BAD_ARG;
    if ((q_rs % 8) || (q_hs % 8) || (o_rs % 2) || (o_hs % 2) || ((uintptr_t)q & 15) || ((uintptr_t)pool & 15) ||
        ((uintptr_t)out & 3))
        return IB_ERR_UNSUPPORTED;
    if (mt < 1 || mt > 4) return IB_ERR_BAD_ARG;
    if (n_entries > 65535) return IB_ERR_TOO_LARGE;
    LatentParams p;
    p.q = (const bf16*)q; p.q_rs = q_rs; p.q_hs = q_hs;
    p.pool = (const bf16*)pool;
    p.out = (bf16*)out; p.o_rs = o_rs; p.o_hs = o_hs;
    p.cu_rows = cu_rows; p.q_start = q_start; p.tables = tables; p.max_blocks = max_blocks;
    p.n_entries = n_entries; p.heads = heads; p.page_size = page_size; p.num_pages = num_pages; p.window = window;
    p.scale = scale; p.splits = splits; p.n_rows_total = n_rows; p.err = err;
    p.part_o = nullptr; p.part_ml = nullptr;
    if (splits > 1) {
        if (!scratch || scratch_bytes < ib_attention_latent_scratch_bytes(n_rows, heads, splits)) return IB_ERR_BAD_ARG;
        p.part_o = (float*)scratch;
        p.part_ml = p.part_o + (size_t)splits * n_rows * heads * KV;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int packed = max_rows_per_entry * heads;
    const int rc = mt == 4 ? launch_latent<2, 2>(p, packed, s)
                 : mt == 3 ? launch_latent<1, 2>(p, packed, s)   // 32 rows in two groups of four warps
                 : mt == 2 ? launch_latent<2, 1>(p, packed, s) : launch_latent<1, 1>(p, packed, s);
    if (rc != IB_OK) return rc;
    if (splits > 1) {
        cudaError_t le = launch_kernel(latent_combine_kernel, dim3(n_rows * heads), dim3(KV >= 256 ? 128 : 64), 0, s,
                                       (const float*)p.part_o, (const float*)p.part_ml, (bf16*)out, o_rs, o_hs,
                                       n_rows, heads, splits);
        if (le != cudaSuccess) return (int)le;
        IB_LAUNCH_CHECK();
    }
    return IB_OK;
}
