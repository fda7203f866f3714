// diff_attention.cu -- differential softmax attention over the paged KV pools for a RAGGED batch (prompt portions and
// single decoded tokens in one launch), plus the append that feeds it.
//
// Per query head two attention maps share one value tensor: the query row holds [map 1 | map 2] (2 * dim values), so
// does the key row of its key/value head; out = rmsnorm_headwise(a1 - lambda * a2) * out_mult, where a_i =
// softmax_i(q_i . k_i * scale) V over the causally visible keys.  The query is first multiplied by a position-dependent
// temperature 1 + coef * ln(floor((p + 1) / every) + 1).  Scores, softmax weights, both weighted sums, the difference
// and the head-wise norm are float; K/V pages are stored in the activation type (float or bfloat16).
//
// Pools: K pages [total_pages][tile_size][2 * dim], V pages [total_pages][tile_size][vdim]; a (slot, kv head, tile)
// entry of the page table names the page of both.  Unmapped pages are skipped, as in the decode kernels.
//
// Work unit: a CTA of 8 warps owns 32 (token, head) rows that read the SAME key/value head: up to 32 / hc consecutive
// tokens of one portion x hc = min(32, heads per kv head) query heads, so every K/V byte staged in shared memory serves
// all of them.  Keys are staged 32 at a time (one key per lane for the scores; lanes switch to value columns for the
// weighted sums).  Long contexts with few CTAs are cut along the keys into `nsplit` parts whose (m, l, acc) partials a
// second kernel merges before the difference and the norm are taken.
#include "seq_common.cuh"

namespace pa {

constexpr int kDaRows = 32;     // (token, head) rows per CTA
constexpr int kDaWarps = 8;
constexpr int kDaRpw = kDaRows / kDaWarps;
constexpr int kDaKeys = 32;     // keys staged per step

struct DiffAttnParams {
    const void* q;              // rows of the projection buffer; the query of head h starts at q_off + h * 2 * dim
    int64_t q_stride;
    int q_off;
    const void* k_pool;
    const void* v_pool;
    const int32_t* table;
    int num_slots, num_kv_heads, num_tiles, total_pages, tile_size;
    const int32_t* tiles;       // [ntiles][4]: first row, tokens, slot, position of the first token
    int heads, dim, vdim;
    float scale, temp_coef;
    int temp_every;
    float lambda, out_mult, eps;
    void* out;                  // [rows][heads * vdim]
    int nsplit;
    float* partial;             // nsplit > 1: [(tile, y, split, row)][4 + 2 * vdim]
    int head_rows;              // tensor-core kernel: every tile is ONE token and the rows are the heads of a kv head
};

__device__ __forceinline__ void da_geometry(int heads, int kv_heads, int& hpg, int& hc, int& nchunk) {
    hpg = heads / kv_heads;
    hc = hpg < kDaRows ? hpg : kDaRows;
    nchunk = (hpg + hc - 1) / hc;
}

template <typename T>
__global__ void kv_append_rows_kernel(T* __restrict__ k_pool, T* __restrict__ v_pool, const int32_t* __restrict__ table,
                                      int num_slots, int num_kv_heads, int num_tiles, int total_pages, int tile_size,
                                      int k_dim, int v_dim, const T* __restrict__ src, int64_t src_stride, int k_off,
                                      int v_off, const int32_t* __restrict__ row_slot,
                                      const int32_t* __restrict__ row_pos, int rows) {
    const int lane = threadIdx.x & 31;
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= (int64_t)rows * num_kv_heads) return;
    const int g = (int)(w % num_kv_heads);
    const int r = (int)(w / num_kv_heads);
    const int slot = row_slot[r], pos = row_pos[r];
    if (pos < 0 || pos / tile_size >= num_tiles || (unsigned)slot >= (unsigned)num_slots) return;
    const int page = table[((int64_t)slot * num_kv_heads + g) * num_tiles + pos / tile_size];
    if (page < 0 || page >= total_pages) return;
    const int64_t prow = (int64_t)page * tile_size + pos % tile_size;
    const T* sk = src + (int64_t)r * src_stride + k_off + (int64_t)g * k_dim;
    const T* sv = src + (int64_t)r * src_stride + v_off + (int64_t)g * v_dim;
    for (int d = lane; d < k_dim; d += 32) k_pool[prow * k_dim + d] = sk[d];
    for (int d = lane; d < v_dim; d += 32) v_pool[prow * v_dim + d] = sv[d];
}

// Difference of the two maps, head-wise RMS norm and the output factor for one row held across a warp: slot i of a lane
// is value column lane + 32 i (PACKED false) or lane * NV + i (PACKED true).
template <int NV, bool PACKED>
__device__ __forceinline__ int da_col(int lane, int i) { return PACKED ? lane * NV + i : lane + 32 * i; }

template <typename T, int NV, bool PACKED = false>
__device__ __forceinline__ void da_finish_row(const float (&a1)[NV], const float (&a2)[NV], float l1, float l2,
                                              const DiffAttnParams& p, int lane, T* __restrict__ dst) {
    float o[NV];
    float ss = 0.f;
    const float i1 = 1.0f / l1, i2 = 1.0f / l2;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const bool ok = da_col<NV, PACKED>(lane, i) < p.vdim;
        o[i] = ok ? a1[i] * i1 - p.lambda * (a2[i] * i2) : 0.f;
        ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)p.vdim + p.eps);
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (da_col<NV, PACKED>(lane, i) < p.vdim) dst[da_col<NV, PACKED>(lane, i)] = from_f32<T>(o[i] * rn * p.out_mult);
}

template <typename T, int NV>
__global__ void __launch_bounds__(kDaWarps * 32) diff_attention_kernel(const DiffAttnParams p) {
    extern __shared__ float smem[];
    const int kd = 2 * p.dim, kds = kd + 1;
    float* Qs = smem;                              // [32][kd]
    float* Ks = Qs + kDaRows * kd;                 // [32][kd + 1]
    float* Vs = Ks + kDaKeys * kds;                // [32][vdim]
    __shared__ int64_t page_row[kDaKeys];          // first pool row of the staged key's page entry, or -1

    int hpg, hc, nchunk;
    da_geometry(p.heads, p.num_kv_heads, hpg, hc, nchunk);
    const int bq = kDaRows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1], slot = tile[2], pos0 = tile[3];
    const int g = blockIdx.y / nchunk, chunk = blockIdx.y % nchunk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);

    // ---- queries: temperature applied in float
    for (int idx = threadIdx.x; idx < kDaRows * kd; idx += blockDim.x) {
        const int r = idx / kd, d = idx % kd;
        const int tok = r / hc, hh = chunk * hc + r % hc;
        float v = 0.f;
        if (tok < bq && tok < ntok && hh < hpg) {
            const int pos = pos0 + tok;
            const float temp = 1.0f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.0f);
            const T* qr = static_cast<const T*>(p.q) + (int64_t)(row0 + tok) * p.q_stride + p.q_off +
                          (int64_t)(g * hpg + hh) * kd;
            v = to_f32<T>(qr[d]) * temp;
        }
        Qs[idx] = v;
    }

    int rpos[kDaRpw];       // last visible key of the row, -1 for an unused row
    float m1[kDaRpw], l1[kDaRpw], m2[kDaRpw], l2[kDaRpw];
    float a1[kDaRpw][NV], a2[kDaRpw][NV];
#pragma unroll
    for (int r = 0; r < kDaRpw; ++r) {
        const int row = warp * kDaRpw + r;
        const int tok = row / hc, hh = chunk * hc + row % hc;
        rpos[r] = (tok < bq && tok < ntok && hh < hpg) ? pos0 + tok : -1;
        m1[r] = m2[r] = -INFINITY;
        l1[r] = l2[r] = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) a1[r][i] = a2[r][i] = 0.f;
    }

    const int total = pos0 + ntok;                       // keys any row of the tile may see
    const int nsteps = (total + kDaKeys - 1) / kDaKeys;
    const int per = (nsteps + p.nsplit - 1) / p.nsplit;
    const int s_begin = blockIdx.z * per, s_end = min(nsteps, s_begin + per);

    for (int st = s_begin; st < s_end; ++st) {
        const int c0 = st * kDaKeys;
        __syncthreads();                                 // the previous step's tiles are consumed (and Qs is written)
        if (threadIdx.x < kDaKeys) {
            const int j = c0 + threadIdx.x;
            int64_t pr = -1;
            if (j < total && j / p.tile_size < p.num_tiles) {
                const int page = p.table[((int64_t)slot * p.num_kv_heads + g) * p.num_tiles + j / p.tile_size];
                if (page >= 0 && page < p.total_pages) pr = (int64_t)page * p.tile_size + j % p.tile_size;
            }
            page_row[threadIdx.x] = pr;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < kDaKeys * kd; idx += blockDim.x) {
            const int key = idx / kd, d = idx % kd;
            const int64_t pr = page_row[key];
            Ks[key * kds + d] = pr >= 0 ? to_f32<T>(kp[pr * kd + d]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < kDaKeys * p.vdim; idx += blockDim.x) {
            const int key = idx / p.vdim, d = idx % p.vdim;
            const int64_t pr = page_row[key];
            Vs[idx] = pr >= 0 ? to_f32<T>(vp[pr * p.vdim + d]) : 0.f;
        }
        __syncthreads();

        // ---- scores: lane = key
        float s1[kDaRpw], s2[kDaRpw];
#pragma unroll
        for (int r = 0; r < kDaRpw; ++r) s1[r] = s2[r] = 0.f;
        const float* kr = Ks + lane * kds;
        const float* qb = Qs + warp * kDaRpw * kd;
        for (int d = 0; d < p.dim; ++d) {
            const float k1 = kr[d], k2 = kr[p.dim + d];
#pragma unroll
            for (int r = 0; r < kDaRpw; ++r) {
                s1[r] = fmaf(qb[r * kd + d], k1, s1[r]);
                s2[r] = fmaf(qb[r * kd + p.dim + d], k2, s2[r]);
            }
        }
        const int j = c0 + lane;
        const bool mapped = page_row[lane] >= 0;
        float p1[kDaRpw], p2[kDaRpw];
#pragma unroll
        for (int r = 0; r < kDaRpw; ++r) {
            const bool vis = mapped && j <= rpos[r];
            const float v1 = vis ? s1[r] * p.scale : -INFINITY, v2 = vis ? s2[r] * p.scale : -INFINITY;
            const float n1 = fmaxf(m1[r], warp_max(v1)), n2 = fmaxf(m2[r], warp_max(v2));
            const float c1 = n1 == -INFINITY ? 1.f : expf(m1[r] - n1), c2 = n2 == -INFINITY ? 1.f : expf(m2[r] - n2);
            p1[r] = vis ? expf(v1 - n1) : 0.f;
            p2[r] = vis ? expf(v2 - n2) : 0.f;
            l1[r] = l1[r] * c1 + warp_sum(p1[r]);
            l2[r] = l2[r] * c2 + warp_sum(p2[r]);
            m1[r] = n1;
            m2[r] = n2;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                a1[r][i] *= c1;
                a2[r][i] *= c2;
            }
        }
        // ---- weighted sums: lane = value column
        const int nk = min(kDaKeys, total - c0);
        for (int jj = 0; jj < nk; ++jj) {
            float v[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < p.vdim ? Vs[jj * p.vdim + lane + 32 * i] : 0.f;
#pragma unroll
            for (int r = 0; r < kDaRpw; ++r) {
                const float w1 = __shfl_sync(0xffffffffu, p1[r], jj), w2 = __shfl_sync(0xffffffffu, p2[r], jj);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    a1[r][i] = fmaf(w1, v[i], a1[r][i]);
                    a2[r][i] = fmaf(w2, v[i], a2[r][i]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kDaRpw; ++r) {
        const int row = warp * kDaRpw + r;
        if (p.nsplit > 1) {
            float* dst = p.partial + ((((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit + blockIdx.z) * kDaRows + row) *
                                         (4 + 2 * p.vdim);
            if (lane == 0) {
                dst[0] = m1[r]; dst[1] = l1[r]; dst[2] = m2[r]; dst[3] = l2[r];
            }
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < p.vdim) {
                    dst[4 + lane + 32 * i] = a1[r][i];
                    dst[4 + p.vdim + lane + 32 * i] = a2[r][i];
                }
        } else if (rpos[r] >= 0) {
            const int tok = row / hc, hh = chunk * hc + row % hc;
            T* dst = static_cast<T*>(p.out) + (int64_t)(row0 + tok) * p.heads * p.vdim + (int64_t)(g * hpg + hh) * p.vdim;
            da_finish_row<T, NV>(a1[r], a2[r], l1[r], l2[r], p, lane, dst);
        }
    }
}

template <typename T, int NV>
__global__ void __launch_bounds__(kDaWarps * 32) diff_attention_merge_kernel(const DiffAttnParams p) {
    int hpg, hc, nchunk;
    da_geometry(p.heads, p.num_kv_heads, hpg, hc, nchunk);
    const int bq = kDaRows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1];
    const int g = blockIdx.y / nchunk, chunk = blockIdx.y % nchunk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = 0; r < kDaRpw; ++r) {
        const int row = warp * kDaRpw + r;
        const int tok = row / hc, hh = chunk * hc + row % hc;
        if (!(tok < bq && tok < ntok && hh < hpg)) continue;
        const float* base = p.partial + (((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit * kDaRows + row) * (4 + 2 * p.vdim);
        const int64_t zs = (int64_t)kDaRows * (4 + 2 * p.vdim);
        float M1 = -INFINITY, M2 = -INFINITY;
        for (int z = 0; z < p.nsplit; ++z) {
            M1 = fmaxf(M1, base[z * zs + 0]);
            M2 = fmaxf(M2, base[z * zs + 2]);
        }
        float l1 = 0.f, l2 = 0.f, a1[NV], a2[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) a1[i] = a2[i] = 0.f;
        for (int z = 0; z < p.nsplit; ++z) {
            const float* pz = base + z * zs;
            const float w1 = pz[0] == -INFINITY ? 0.f : expf(pz[0] - M1), w2 = pz[2] == -INFINITY ? 0.f : expf(pz[2] - M2);
            l1 = fmaf(w1, pz[1], l1);
            l2 = fmaf(w2, pz[3], l2);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < p.vdim) {
                    a1[i] = fmaf(w1, pz[4 + lane + 32 * i], a1[i]);
                    a2[i] = fmaf(w2, pz[4 + p.vdim + lane + 32 * i], a2[i]);
                }
        }
        T* dst = static_cast<T*>(p.out) + (int64_t)(row0 + tok) * p.heads * p.vdim + (int64_t)(g * hpg + hh) * p.vdim;
        da_finish_row<T, NV>(a1, a2, l1, l2, p, lane, dst);
    }
}


// ---- single-token tiles (decode) ------------------------------------------------------------------------------------
// One CTA = one token x one key/value head x one part of the context; its R >= heads-per-kv-head rows are the query
// heads of the group.  Nothing is staged: each of the 8 warps takes every 8th run of 32 keys, a lane reads ITS key's row
// with 16-byte loads straight into the two dot products of every row (queries broadcast from shared memory), the warp
// does the online softmax, then lanes switch to value columns and read each key's value row coalesced.  The 8 warps'
// (m, l, acc) are merged through shared memory; nsplit > 1 leaves the CTA's partial for diff_attention_merge_kernel.
// Needs dim a multiple of the 16-byte vector and R * NV <= 32 (the dispatcher falls back to the tile kernel otherwise).
template <typename T> struct DaVec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void da_load16(const T* __restrict__ p, float (&f)[DaVec<T>::N]) {
    const uint4 v = ldg_stream_128(p);
    if (sizeof(T) == 4) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    } else {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}

// NV consecutive values of a row starting at element lane * NV (NV * sizeof(T) is 4, 8, 16 or 32 bytes)
template <typename T, int NV>
__device__ __forceinline__ void da_load_packed(const T* __restrict__ p, float (&f)[NV]) {
    constexpr int BYTES = NV * sizeof(T);
    if (BYTES >= 16) {
#pragma unroll
        for (int c = 0; c < BYTES / 16; ++c) {
            float t[DaVec<T>::N];
            da_load16<T>(p + c * DaVec<T>::N, t);
#pragma unroll
            for (int i = 0; i < DaVec<T>::N; ++i) f[c * DaVec<T>::N + i] = t[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) f[i] = to_f32<T>(p[i]);
    }
}

template <typename T, int R, int NV, bool PACKED>
__global__ void __launch_bounds__(kDaWarps * 32) diff_attention_decode_kernel(const DiffAttnParams p) {
    extern __shared__ float smem[];
    constexpr int VN = DaVec<T>::N;
    const int kd = 2 * p.dim;
    float* Qs = smem;                                   // [R][kd]
    float* Ps = Qs + R * kd;                            // [warps][R][4 + 2 * vdim]
    const int pstride = 4 + 2 * p.vdim;
    const int hpg = p.heads / p.num_kv_heads;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], slot = tile[2], pos = tile[3];
    const int g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);
    {
        const float temp = 1.0f + p.temp_coef * logf((float)((pos + 1) / p.temp_every) + 1.0f);
        for (int idx = threadIdx.x; idx < R * kd; idx += blockDim.x) {
            const int r = idx / kd, d = idx % kd;
            float v = 0.f;
            if (r < hpg)
                v = to_f32<T>(static_cast<const T*>(p.q)[(int64_t)row0 * p.q_stride + p.q_off + (int64_t)(g * hpg + r) * kd + d]) * temp;
            Qs[idx] = v;
        }
    }
    __syncthreads();
    float m1[R], l1[R], m2[R], l2[R], a1[R][NV], a2[R][NV];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m1[r] = m2[r] = -INFINITY;
        l1[r] = l2[r] = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) a1[r][i] = a2[r][i] = 0.f;
    }
    const int total = pos + 1;
    const int nsteps = (total + kDaKeys - 1) / kDaKeys;
    const int per = (nsteps + p.nsplit - 1) / p.nsplit;
    const int s_begin = blockIdx.z * per, s_end = min(nsteps, s_begin + per);
    const int32_t* trow = p.table + ((int64_t)slot * p.num_kv_heads + g) * p.num_tiles;
    for (int st = s_begin + warp; st < s_end; st += kDaWarps) {
        const int j = st * kDaKeys + lane;
        int prow = -1;                                  // pool row of this lane's key
        if (j < total && j / p.tile_size < p.num_tiles) {
            const int page = trow[j / p.tile_size];
            if (page >= 0 && page < p.total_pages) prow = page * p.tile_size + j % p.tile_size;
        }
        float s1[R], s2[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s1[r] = s2[r] = 0.f;
        if (prow >= 0) {
            const T* kr = kp + (int64_t)prow * kd;
#pragma unroll 2
            for (int d0 = 0; d0 < p.dim; d0 += VN) {
                float k1[VN], k2[VN];
                da_load16<T>(kr + d0, k1);
                da_load16<T>(kr + p.dim + d0, k2);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float* q1 = Qs + r * kd + d0;
                    const float* q2 = q1 + p.dim;
#pragma unroll
                    for (int i = 0; i < VN; ++i) {
                        s1[r] = fmaf(q1[i], k1[i], s1[r]);
                        s2[r] = fmaf(q2[i], k2[i], s2[r]);
                    }
                }
            }
        }
        const bool vis = prow >= 0;
        float p1[R], p2[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float v1 = vis ? s1[r] * p.scale : -INFINITY, v2 = vis ? s2[r] * p.scale : -INFINITY;
            const float n1 = fmaxf(m1[r], warp_max(v1)), n2 = fmaxf(m2[r], warp_max(v2));
            const float c1 = n1 == -INFINITY ? 1.f : expf(m1[r] - n1), c2 = n2 == -INFINITY ? 1.f : expf(m2[r] - n2);
            p1[r] = vis ? expf(v1 - n1) : 0.f;
            p2[r] = vis ? expf(v2 - n2) : 0.f;
            l1[r] = l1[r] * c1 + warp_sum(p1[r]);
            l2[r] = l2[r] * c2 + warp_sum(p2[r]);
            m1[r] = n1;
            m2[r] = n2;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                a1[r][i] *= c1;
                a2[r][i] *= c2;
            }
        }
        const int nk = min(kDaKeys, total - st * kDaKeys);
#pragma unroll 4
        for (int jj = 0; jj < nk; ++jj) {
            const int pr = __shfl_sync(0xffffffffu, prow, jj);
            float v[NV];
            if (pr >= 0) {
                const T* vr = vp + (int64_t)pr * p.vdim;
                if (PACKED) {
                    da_load_packed<T, NV>(vr + lane * NV, v);
                } else {
#pragma unroll
                    for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < p.vdim ? to_f32<T>(vr[lane + 32 * i]) : 0.f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < NV; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float w1 = __shfl_sync(0xffffffffu, p1[r], jj), w2 = __shfl_sync(0xffffffffu, p2[r], jj);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    a1[r][i] = fmaf(w1, v[i], a1[r][i]);
                    a2[r][i] = fmaf(w2, v[i], a2[r][i]);
                }
            }
        }
    }
    // ---- the warps' partials -> shared memory, merged by warp r for row r
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float* dst = Ps + ((int64_t)warp * R + r) * pstride;
        if (lane == 0) {
            dst[0] = m1[r]; dst[1] = l1[r]; dst[2] = m2[r]; dst[3] = l2[r];
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = da_col<NV, PACKED>(lane, i);
            if (c < p.vdim) {
                dst[4 + c] = a1[r][i];
                dst[4 + p.vdim + c] = a2[r][i];
            }
        }
    }
    __syncthreads();
    for (int r = warp; r < R; r += kDaWarps) {
        if (r >= hpg) continue;
        float M1 = -INFINITY, M2 = -INFINITY;
        for (int w = 0; w < kDaWarps; ++w) {
            M1 = fmaxf(M1, Ps[((int64_t)w * R + r) * pstride + 0]);
            M2 = fmaxf(M2, Ps[((int64_t)w * R + r) * pstride + 2]);
        }
        float L1 = 0.f, L2 = 0.f, b1[NV], b2[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) b1[i] = b2[i] = 0.f;
        for (int w = 0; w < kDaWarps; ++w) {
            const float* pw = Ps + ((int64_t)w * R + r) * pstride;
            const float w1 = pw[0] == -INFINITY ? 0.f : expf(pw[0] - M1), w2 = pw[2] == -INFINITY ? 0.f : expf(pw[2] - M2);
            L1 = fmaf(w1, pw[1], L1);
            L2 = fmaf(w2, pw[3], L2);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = da_col<NV, PACKED>(lane, i);
                if (c < p.vdim) {
                    b1[i] = fmaf(w1, pw[4 + c], b1[i]);
                    b2[i] = fmaf(w2, pw[4 + p.vdim + c], b2[i]);
                }
            }
        }
        if (p.nsplit > 1) {
            float* dst = p.partial + ((((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit + blockIdx.z) * kDaRows + r) * pstride;
            if (lane == 0) {
                dst[0] = M1; dst[1] = L1; dst[2] = M2; dst[3] = L2;
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = da_col<NV, PACKED>(lane, i);
                if (c < p.vdim) {
                    dst[4 + c] = b1[i];
                    dst[4 + p.vdim + c] = b2[i];
                }
            }
        } else {
            T* dst = static_cast<T*>(p.out) + (int64_t)row0 * p.heads * p.vdim + (int64_t)(g * hpg + r) * p.vdim;
            da_finish_row<T, NV, PACKED>(b1, b2, L1, L2, p, lane, dst);
        }
    }
}

template <typename T, int R, int NV>
static int da_decode_launch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    const size_t smem = ((size_t)R * 2 * p.dim + (size_t)kDaWarps * R * (4 + 2 * p.vdim)) * sizeof(float);
    if (smem > 200 * 1024) return PA_ERR_UNSUPPORTED;
    const bool packed = p.vdim == 32 * NV && (NV * sizeof(T)) % 4 == 0 && (NV * sizeof(T) <= 16 || (NV * sizeof(T)) % 16 == 0);
    auto kern = packed ? diff_attention_decode_kernel<T, R, NV, true> : diff_attention_decode_kernel<T, R, NV, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)p.num_kv_heads, (unsigned)p.nsplit);
    kern<<<grid, kDaWarps * 32, smem, st>>>(p);
    if (p.nsplit > 1) {
        dim3 g2((unsigned)ntiles, (unsigned)p.num_kv_heads);
        diff_attention_merge_kernel<T, NV><<<g2, kDaWarps * 32, 0, st>>>(p);
    }
    PA_RETURN_LAUNCH_STATUS();
}

// PA_ERR_UNSUPPORTED: this shape stays on the tile kernel
template <typename T>
static int da_decode_dispatch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    const int hpg = p.heads / p.num_kv_heads, nv = (p.vdim + 31) / 32;
    if (p.dim % DaVec<T>::N || hpg > 8 || nv > 8) return PA_ERR_UNSUPPORTED;
    if ((uintptr_t)p.k_pool % 16 || (uintptr_t)p.v_pool % 16) return PA_ERR_UNSUPPORTED;
    const int NVc = nv <= 1 ? 1 : nv <= 2 ? 2 : nv <= 4 ? 4 : 8;
    if (hpg <= 4) {
        switch (NVc) {
            case 1: return da_decode_launch<T, 4, 1>(p, ntiles, st);
            case 2: return da_decode_launch<T, 4, 2>(p, ntiles, st);
            case 4: return da_decode_launch<T, 4, 4>(p, ntiles, st);
            default: return da_decode_launch<T, 4, 8>(p, ntiles, st);
        }
    }
    switch (NVc) {
        case 1: return da_decode_launch<T, 8, 1>(p, ntiles, st);
        case 2: return da_decode_launch<T, 8, 2>(p, ntiles, st);
        case 4: return da_decode_launch<T, 8, 4>(p, ntiles, st);
        default: return PA_ERR_UNSUPPORTED;
    }
}

template <typename T, int NV>
static int da_launch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    int hpg = p.heads / p.num_kv_heads;
    int hc = hpg < kDaRows ? hpg : kDaRows;
    int nchunk = (hpg + hc - 1) / hc;
    const size_t smem = ((size_t)kDaRows * 2 * p.dim + (size_t)kDaKeys * (2 * p.dim + 1) + (size_t)kDaKeys * p.vdim) * sizeof(float);
    if (smem > 200 * 1024) return PA_ERR_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(diff_attention_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)(p.num_kv_heads * nchunk), (unsigned)p.nsplit);
    diff_attention_kernel<T, NV><<<grid, kDaWarps * 32, smem, st>>>(p);
    if (p.nsplit > 1) {
        dim3 g2((unsigned)ntiles, (unsigned)(p.num_kv_heads * nchunk));
        diff_attention_merge_kernel<T, NV><<<g2, kDaWarps * 32, 0, st>>>(p);
    }
    PA_RETURN_LAUNCH_STATUS();
}

template <typename T>
static int da_dispatch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    const int nv = (p.vdim + 31) / 32;
    switch (nv) {
        case 1: return da_launch<T, 1>(p, ntiles, st);
        case 2: return da_launch<T, 2>(p, ntiles, st);
        case 3: return da_launch<T, 3>(p, ntiles, st);
        case 4: return da_launch<T, 4>(p, ntiles, st);
        case 5: case 6: return da_launch<T, 6>(p, ntiles, st);
        case 7: case 8: return da_launch<T, 8>(p, ntiles, st);
        default: return PA_ERR_UNSUPPORTED;
    }
}

// ---- prompt portions on the tensor cores (bfloat16) -------------------------------------------------------------------
// One CTA = up to 64 consecutive tokens of one portion x ONE query head; 8 warps: warp w owns the 16 rows (w & 3) of
// map (w >> 2), so each map is a flash-attention of its own (mma.sync m16n8k16, bfloat16 operands, float accumulators)
// over the SAME staged key and value tiles: 64 keys per step, located through the page table and brought in with
// 16-byte cp.async copies into two buffers (the copies of step t + 1 fly while step t is multiplied).  Rows are padded
// by 16 bytes so that ldmatrix reads are conflict-free.  The dot products are raw q . k; the position-dependent query
// temperature and the scale multiply the float score (same product, no second rounding of q).  Scores, the running
// maximum, the exponentials and their sum are float; the weights enter the second product rounded to bfloat16, like
// every other matrix operand of this precision.  At the end the warps of map 2 leave a2 in shared memory and the warps
// of map 1 take the difference, the head-wise norm and the output factor.
// DIM and VDIM are the PADDED sizes (32, 64 or 128): a map's dim values (any multiple of 8 up to DIM) sit at the start
// of its DIM columns in shared memory and the rest is zero, likewise the value columns; 16-wide steps that are all
// padding are skipped.
// head_rows (decoded tokens, many sequences in the batch): a tile is ONE token, the CTA's rows are the query heads that
// share key/value head blockIdx.y, all at the token's position, so a key/value byte is staged once for the whole group
// and the dot products of every head with it are one MMA.  Up to 16 heads per key/value head: the four warps of a map
// split the keys of a step; more: warps whose 16 rows hold no head only help to copy.
constexpr int kDmRows = 64, kDmKeys = 64, kDmThreads = 256, kDmPad = 8;
static_assert(kDmThreads == 4 * kDmKeys, "four copying threads per key");

// NST key/value buffers form a ring with NST - 1 steps of copies in flight; QR query rows are staged.  Prompt portions:
// <2, 64> (the arithmetic of a step hides the next step's copies).  Head rows with at most 16 heads per key/value head:
// <3, 16> -- one 16-row MMA group is all the arithmetic there is, so the copies of two steps must be in flight, and the
// small query tile leaves room for two such CTAs per SM.
template <int DIM, int VDIM, int NST, int QR>
__global__ void __launch_bounds__(kDmThreads, 2) diff_attention_mma_kernel(const DiffAttnParams p) {
    constexpr int KD = 2 * DIM, KS = KD + kDmPad, VS = VDIM + kDmPad, NT = VDIM / 8;
    extern __shared__ __align__(16) unsigned char dm_smem[];
    bf16_t* Qs = reinterpret_cast<bf16_t*>(dm_smem);        // [QR][KS]
    bf16_t* Ks = Qs + QR * KS;                               // [NST][64][KS]
    bf16_t* Vs = Ks + NST * kDmKeys * KS;                    // [NST][64][VS]
    __shared__ int key_ok[NST][kDmKeys];

    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], slot = tile[2], pos0 = tile[3];
    const int hpg = p.heads / p.num_kv_heads;
    const bool hr = p.head_rows != 0;
    const int ntok = hr ? hpg : tile[1];                     // rows of the CTA that hold a query
    const int g = hr ? blockIdx.y : blockIdx.y / hpg;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp & 3, map = warp >> 2;
    // QR == 16 (head rows, one 16-row group): the four warps of a map SPLIT the 64 keys of a step, 16 each, over the
    // same rows, and their (m, l, o) meet in shared memory at the end; else a warp owns 16 rows and takes all 64 keys.
    constexpr bool KSPLIT = QR == 16;
    constexpr int NKG = KSPLIT ? 1 : 4;                      // groups of 16 keys a warp takes per step
    const int kg0 = KSPLIT ? rg : 0, rbase = KSPLIT ? 0 : rg * 16;
    const bool active = KSPLIT || rg * 16 < ntok;            // this warp has rows with a query
    auto q_row = [&](int r) -> int64_t { return hr ? row0 : row0 + r; };             // token row of CTA row r
    auto q_head = [&](int r) -> int { return hr ? g * hpg + r : (int)blockIdx.y; };   // its query head
    const bf16_t* kp = static_cast<const bf16_t*>(p.k_pool);
    const bf16_t* vp = static_cast<const bf16_t*>(p.v_pool);
    const int32_t* trow = p.table + ((int64_t)slot * p.num_kv_heads + g) * p.num_tiles;
    const int total = pos0 + (hr ? 1 : ntok);                // keys any row of the tile may see
    const int nkt = (total + kDmKeys - 1) / kDmKeys;
    const int dim = p.dim, vdim = p.vdim, kd = 2 * dim;      // the real sizes

    for (int c = tid; c < QR * (KD / 8); c += kDmThreads) {
        const int r = c / (KD / 8), v = c % (KD / 8), mp = v / (DIM / 8), cv = (v % (DIM / 8)) * 8;
        const bool ok = r < ntok && cv < dim;
        const bf16_t* src = static_cast<const bf16_t*>(p.q) +
                            (ok ? q_row(r) * p.q_stride + p.q_off + (int64_t)q_head(r) * kd + mp * dim + cv : 0);
        cp_async_16(smem_u32(Qs + r * KS + v * 8), src, ok);
    }
    auto pool_row = [&](int j) -> int64_t {
        if (j < total && j / p.tile_size < p.num_tiles) {
            const int page = trow[j / p.tile_size];
            if (page >= 0 && page < p.total_pages) return (int64_t)page * p.tile_size + j % p.tile_size;
        }
        return -1;
    };
    // four threads per key: ONE page look-up per thread and step; a thread copies every fourth 16-byte piece of its
    // key's row and of its value row (the four threads of a key cover 64 contiguous bytes per instruction)
    auto load_tile = [&](int kt, int buf) {
        const int key = tid >> 2, q4 = tid & 3;
        const int64_t pr = pool_row(kt * kDmKeys + key);
        if (q4 == 0) key_ok[buf][key] = pr >= 0;
        bf16_t* kdst = Ks + (buf * kDmKeys + key) * KS;
        const bf16_t* ksrc = kp + (pr >= 0 ? pr * kd : 0);
#pragma unroll
        for (int i = 0; i < KD / 32; ++i) {
            const int v = q4 + 4 * i, mp = v / (DIM / 8), cv = (v % (DIM / 8)) * 8;
            const bool ok = pr >= 0 && cv < dim;
            cp_async_16(smem_u32(kdst + v * 8), ok ? ksrc + mp * dim + cv : kp, ok);
        }
        bf16_t* vdst = Vs + (buf * kDmKeys + key) * VS;
        const bf16_t* vsrc = vp + (pr >= 0 ? pr * vdim : 0);
#pragma unroll
        for (int i = 0; i < VDIM / 32; ++i) {
            const int v = q4 + 4 * i;
            const bool ok = pr >= 0 && v * 8 < vdim;
            cp_async_16(smem_u32(vdst + v * 8), ok ? vsrc + v * 8 : vp, ok);
        }
    };
#pragma unroll
    for (int t = 0; t < NST - 1; ++t) {
        if (t < nkt) load_tile(t, t);
        cp_async_commit();
    }

    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[t][c] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int rpos[2];
    float sc[2];                                             // scale * temperature * log2(e) of the thread's two rows
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        rpos[i] = pos0 + (hr ? 0 : rbase + (lane >> 2) + 8 * i);
        sc[i] = p.scale * (1.0f + p.temp_coef * logf((float)((rpos[i] + 1) / p.temp_every) + 1.0f)) * 1.4426950408889634f;
    }

    for (int kt = 0; kt < nkt; ++kt) {
        const int buf = kt % NST, c0 = kt * kDmKeys;
        if (kt + NST - 1 < nkt) load_tile(kt + NST - 1, (kt + NST - 1) % NST);
        cp_async_commit();
        cp_async_wait<NST - 1>();
        __syncthreads();
        if (active) {
        float s[2 * NKG][4];
#pragma unroll
        for (int t = 0; t < 2 * NKG; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) s[t][c] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DIM; ks += 16) {
            if (ks >= dim) continue;                         // all padding
            uint32_t a[4];
            ldsm_x4(smem_u32(Qs + (rbase + (lane & 15)) * KS + map * DIM + ks + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int np = 0; np < NKG; ++np) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(Ks + (buf * kDmKeys + (kg0 + np) * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + map * DIM + ks +
                                 ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
                mma_bf16_16816(s[2 * np], a, b0, b1);
                mma_bf16_16816(s[2 * np + 1], a, b2, b3);
            }
        }
        // ---- float scores -> weights (log2 domain)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int t = 0; t < 2 * NKG; ++t) {
            const int col = (2 * kg0 + t) * 8 + 2 * (lane & 3);
            const int2 okk = *reinterpret_cast<const int2*>(&key_ok[buf][col]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = c >> 1;
                const bool vis = ((c & 1) ? okk.y : okk.x) && c0 + col + (c & 1) <= rpos[i];
                s[t][c] = vis ? s[t][c] * sc[i] : -INFINITY;
                mx[i] = fmaxf(mx[i], s[t][c]);
            }
        }
        float ref[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float mn = fmaxf(m[i], mx[i]);
            ref[i] = mn == -INFINITY ? 0.f : mn;
            const float corr = exp2f(m[i] - ref[i]);         // m = -inf: 0 (nothing accumulated yet)
            m[i] = mn;
            l[i] *= corr;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                o[t][2 * i] *= corr;
                o[t][2 * i + 1] *= corr;
            }
        }
#pragma unroll
        for (int t = 0; t < 2 * NKG; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                s[t][c] = exp2f(s[t][c] - ref[c >> 1]);
                l[c >> 1] += s[t][c];
            }
        // ---- weighted sums
#pragma unroll
        for (int kk = 0; kk < NKG; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                if (np * 16 >= vdim) continue;               // all padding
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(smem_u32(Vs + (buf * kDmKeys + (kg0 + kk) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + np * 16 +
                                       (lane >> 4) * 8), b0, b1, b2, b3);
                mma_bf16_16816(o[2 * np], a, b0, b1);
                mma_bf16_16816(o[2 * np + 1], a, b2, b3);
            }
        }
        }
        __syncthreads();                                     // this buffer is free for the copies of step kt + NST
    }
    cp_async_wait<0>();
    // ---- a2 through shared memory, then difference, head-wise norm, output factor
    bool fin = active;                                       // this warp finishes rows
    if (KSPLIT) {
        // [rg][map][lane][m0 m1 l0 l1 o...] over the key / value buffers (odd stride: conflict-free); warp rg == 0 of
        // each map merges the four parts into its registers
        constexpr int PST = 4 + NT * 4 + 1;
        float* Pm = reinterpret_cast<float*>(Ks);
        float* mine = Pm + ((rg * 2 + map) * 32 + lane) * PST;
        mine[0] = m[0]; mine[1] = m[1]; mine[2] = l[0]; mine[3] = l[1];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) mine[4 + t * 4 + c] = o[t][c];
        __syncthreads();
        fin = rg == 0;
        if (fin) {
            float M[2] = {m[0], m[1]};
#pragma unroll
            for (int q = 1; q < 4; ++q) {
                const float* pq = Pm + ((q * 2 + map) * 32 + lane) * PST;
                M[0] = fmaxf(M[0], pq[0]);
                M[1] = fmaxf(M[1], pq[1]);
            }
            float w0[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                w0[i] = m[i] == -INFINITY ? 0.f : exp2f(m[i] - M[i]);
                l[i] *= w0[i];
            }
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[t][c] *= w0[c >> 1];
#pragma unroll
            for (int q = 1; q < 4; ++q) {
                const float* pq = Pm + ((q * 2 + map) * 32 + lane) * PST;
                float wq[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    wq[i] = pq[i] == -INFINITY ? 0.f : exp2f(pq[i] - M[i]);
                    l[i] = fmaf(wq[i], pq[2 + i], l[i]);
                }
#pragma unroll
                for (int t = 0; t < NT; ++t)
#pragma unroll
                    for (int c = 0; c < 4; ++c) o[t][c] = fmaf(wq[c >> 1], pq[4 + t * 4 + c], o[t][c]);
            }
        }
        __syncthreads();                                     // the parts are read: A2 may overwrite them
    }
    float* A2 = reinterpret_cast<float*>(Ks);                // [QR][VDIM] over the key / value buffers
    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        inv[i] = 1.0f / l[i];
    }
    if (map == 1 && fin) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                A2[(rg * 16 + (lane >> 2) + 8 * (c >> 1)) * VDIM + t * 8 + 2 * (lane & 3) + (c & 1)] = o[t][c] * inv[c >> 1];
    }
    __syncthreads();
    if (map == 0 && fin) {
        float ss[2] = {0.f, 0.f};
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float a2 = A2[(rg * 16 + (lane >> 2) + 8 * (c >> 1)) * VDIM + t * 8 + 2 * (lane & 3) + (c & 1)];
                o[t][c] = o[t][c] * inv[c >> 1] - p.lambda * a2;
                ss[c >> 1] = fmaf(o[t][c], o[t][c], ss[c >> 1]);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 1);
            ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 2);
            const int r = rg * 16 + (lane >> 2) + 8 * i;
            if (r >= ntok) continue;
            const float f = p.out_mult / sqrtf(ss[i] / (float)vdim + p.eps);      // padded columns are exactly zero
            bf16_t* dst = static_cast<bf16_t*>(p.out) + q_row(r) * p.heads * vdim + (int64_t)q_head(r) * vdim + 2 * (lane & 3);
#pragma unroll
            for (int t = 0; t < NT; ++t)
                if (t * 8 < vdim) *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16x2(o[t][2 * i] * f, o[t][2 * i + 1] * f);
        }
    }
}

template <int DIM, int VDIM, int NST, int QR>
static int dm_launch_as(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    const size_t smem = ((size_t)(QR + NST * kDmKeys) * (2 * DIM + kDmPad) + (size_t)NST * kDmKeys * (VDIM + kDmPad)) * sizeof(bf16_t);
    auto kern = diff_attention_mma_kernel<DIM, VDIM, NST, QR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)ntiles, (unsigned)(p.head_rows ? p.num_kv_heads : p.heads));
    kern<<<grid, kDmThreads, smem, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

template <int DIM, int VDIM>
static int dm_launch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    if (p.head_rows && p.heads / p.num_kv_heads <= 16) return dm_launch_as<DIM, VDIM, 3, 16>(p, ntiles, st);
    return dm_launch_as<DIM, VDIM, 2, kDmRows>(p, ntiles, st);
}

static bool dm_shape_ok(int dim, int vdim) {
    return dim % 8 == 0 && dim <= 128 && vdim % 8 == 0 && vdim <= 128;
}
static int dm_padded(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : 128; }

// PA_ERR_UNSUPPORTED: this shape or these pointers stay on the float kernel
static int dm_dispatch(const DiffAttnParams& p, int ntiles, cudaStream_t st) {
    if (!dm_shape_ok(p.dim, p.vdim) || p.q_stride % 8 || p.q_off % 8) return PA_ERR_UNSUPPORTED;
    if (p.head_rows && p.heads / p.num_kv_heads > kDmRows) return PA_ERR_UNSUPPORTED;
    if ((uintptr_t)p.q % 16 || (uintptr_t)p.k_pool % 16 || (uintptr_t)p.v_pool % 16 || (uintptr_t)p.out % 4) return PA_ERR_UNSUPPORTED;
    const int dp = dm_padded(p.dim), vp = dm_padded(p.vdim);
#define PA_DM_CASE(D, V) if (dp == D && vp == V) return dm_launch<D, V>(p, ntiles, st)
    PA_DM_CASE(32, 32); PA_DM_CASE(32, 64); PA_DM_CASE(32, 128);
    PA_DM_CASE(64, 32); PA_DM_CASE(64, 64); PA_DM_CASE(64, 128);
    PA_DM_CASE(128, 32); PA_DM_CASE(128, 64); PA_DM_CASE(128, 128);
#undef PA_DM_CASE
    return PA_ERR_UNSUPPORTED;
}

}  // namespace pa

using namespace pa;

PA_API int pa_kv_append_rows(void* d_k_pool, void* d_v_pool, const int32_t* d_table, int num_slots, int num_kv_heads,
                             int num_tiles, int total_pages, int tile_size, int k_dim, int v_dim, const void* d_src,
                             int64_t src_stride, int k_off, int v_off, const int32_t* d_row_slot,
                             const int32_t* d_row_pos, int rows, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_k_pool && d_v_pool && d_table && d_src && d_row_slot && d_row_pos && rows >= 0);
    PA_CHECK_ARG(num_slots > 0 && num_kv_heads > 0 && num_tiles > 0 && total_pages > 0 && tile_size > 0 && k_dim > 0 && v_dim > 0);
    if (rows == 0) return PA_OK;
    const int64_t threads = (int64_t)rows * num_kv_heads * 32;
    PA_DISPATCH_ELEM(elem, kv_append_rows_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<T*>(d_k_pool), static_cast<T*>(d_v_pool), d_table, num_slots, num_kv_heads,
                               num_tiles, total_pages, tile_size, k_dim, v_dim, static_cast<const T*>(d_src), src_stride,
                               k_off, v_off, d_row_slot, d_row_pos, rows));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_diff_attention_tile_tokens(int heads, int kv_heads) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    const int hpg = heads / kv_heads;
    return kDaRows / (hpg < kDaRows ? hpg : kDaRows);
}

PA_API int pa_diff_attention_mma_tile_tokens(int dim, int vdim, int elem) {
    return elem == 2 && dm_shape_ok(dim, vdim) ? kDmRows : 0;
}

PA_API int pa_diff_attention_mma_head_rows(int heads, int kv_heads, int dim, int vdim, int elem) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    return elem == 2 && dm_shape_ok(dim, vdim) && heads / kv_heads <= kDmRows ? 1 : 0;
}

PA_API size_t pa_diff_attention_workspace_bytes(int num_tiles_q, int heads, int kv_heads, int vdim, int nsplit) {
    if (nsplit <= 1 || num_tiles_q <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
    const int hpg = heads / kv_heads, hc = hpg < kDaRows ? hpg : kDaRows, nchunk = (hpg + hc - 1) / hc;
    return (size_t)num_tiles_q * kv_heads * nchunk * nsplit * kDaRows * (4 + 2 * vdim) * sizeof(float);
}

PA_API int pa_diff_attention(const void* d_q, int64_t q_stride, int q_off, const void* d_k_pool, const void* d_v_pool,
                             const int32_t* d_table, int num_slots, int num_kv_heads, int num_tiles, int total_pages,
                             int tile_size, const int32_t* d_q_tiles, int num_q_tiles, int heads, int dim, int vdim,
                             float scale, float temp_coef, int temp_every, float lambda, float out_mult, float eps,
                             void* d_out, int elem, int nsplit, int tile_kind, void* d_workspace,
                             size_t workspace_bytes, pa_stream_t stream) {
    PA_CHECK_ARG(d_q && d_k_pool && d_v_pool && d_table && d_q_tiles && d_out && num_q_tiles >= 0);
    PA_CHECK_ARG(num_slots > 0 && num_kv_heads > 0 && num_tiles > 0 && total_pages > 0 && tile_size > 0);
    PA_CHECK_ARG(heads > 0 && heads % num_kv_heads == 0 && dim > 0 && vdim > 0 && temp_every > 0);
    if (num_q_tiles == 0) return PA_OK;
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 1 && (!d_workspace || workspace_bytes < pa_diff_attention_workspace_bytes(num_q_tiles, heads, num_kv_heads, vdim, nsplit)))
        return PA_ERR_WORKSPACE;
    DiffAttnParams p;
    p.q = d_q; p.q_stride = q_stride; p.q_off = q_off; p.k_pool = d_k_pool; p.v_pool = d_v_pool; p.table = d_table;
    p.num_slots = num_slots; p.num_kv_heads = num_kv_heads; p.num_tiles = num_tiles; p.total_pages = total_pages;
    p.tile_size = tile_size; p.tiles = d_q_tiles; p.heads = heads; p.dim = dim; p.vdim = vdim; p.scale = scale;
    p.temp_coef = temp_coef; p.temp_every = temp_every; p.lambda = lambda; p.out_mult = out_mult; p.eps = eps;
    p.out = d_out; p.nsplit = nsplit; p.partial = static_cast<float*>(d_workspace); p.head_rows = 0;
    if (elem != 4 && elem != 2) return PA_ERR_UNSUPPORTED;
    if (tile_kind == 2 || tile_kind == 3) {   // on the tensor cores: tiles of up to pa_diff_attention_mma_tile_tokens
        if (elem != 2 || nsplit != 1) return PA_ERR_UNSUPPORTED;   // tokens (2), or one token with its heads as rows (3)
        p.head_rows = tile_kind == 3;
        return dm_dispatch(p, num_q_tiles, as_stream(stream));
    }
    if (tile_kind == 1) {       // every tile is one token: the streaming kernel, where it serves the shape
        const int st = elem == 4 ? da_decode_dispatch<float>(p, num_q_tiles, as_stream(stream))
                                 : da_decode_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
        if (st != PA_ERR_UNSUPPORTED) return st;
    }
    if (elem == 4) return da_dispatch<float>(p, num_q_tiles, as_stream(stream));
    return da_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
}
