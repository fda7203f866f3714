// latent_attention.cu -- attention through a low-rank latent (one cached row per token for ALL heads) over a paged pool,
// for a RAGGED batch (prompt portions and single decoded tokens in one launch), and the ops around it.
//
// Per token the pool keeps ONE row [c (kv_rank) | kr (rot_dim)]: c is the normalised latent from which every head's
// keys and values are linear maps (k_h = Wuk_h c, v_h = Wuv_h c), kr a rotated key part shared by all heads.  The maps
// are never applied to the cache.  With q_h = [qp_h | qr_h]:
//
//     score_h(t, j) = (qp_h . Wuk_h c_j + qr_h . kr_j) * scale = ([Wuk_h^T qp_h | qr_h] . [c_j | kr_j]) * scale
//     out_h(t)      = Wuv_h (sum_j p_h(t, j) c_j)
//
// so attention is multi-query attention of the `heads` latent queries ql_h = Wuk_h^T qp_h (kv_rank wide, next to the
// rotated part) against the pool rows, whose first kv_rank columns are also the values; Wuk^T before and Wuv after are
// per-head matrix products over the batch rows (head_linear_kernel).  Scores, softmax weights and the weighted sums are
// float; pool rows are stored in the activation type (float or bfloat16).
//
//   rope_table_kernel        cos / sin of p * base^(-2i / dims) per batch row (angles in double, table in float)
//   rope_rows_kernel         in-place rotation of interleaved pairs (2i, 2i + 1) of every head's rotated part
//   latent_kv_append_kernel  RMS norm (per-channel gain) of the latent columns + rotation of the shared key part, written
//                            to the row's place in the pool
//   head_linear_kernel       out[r, h, :] = x[r, h, :] . W[h]  (W [heads][K][N]), any strides
//   latent_attention_kernel  float tile kernel, any shape, keys optionally split with a merge kernel
//   latent_attention_mma_kernel  bfloat16 tensor-core kernel (mma.sync), see there
//   head_gate_kernel         out[r, h * vdim + v] = in[r, h, v] * sigmoid(gate[r, h])
#include "seq_common.cuh"

namespace pa {

// ---- rotation -------------------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int32_t* __restrict__ row_pos, int rows, int dims, double log_base,
                                  float* __restrict__ table) {
    const int half = dims / 2;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * half) return;
    const int r = (int)(i / half), k = (int)(i % half);
    const double a = (double)row_pos[r] * exp(-2.0 * (double)k / (double)dims * log_base);
    double s, c;
    sincos(a, &s, &c);
    table[2 * i] = (float)c;
    table[2 * i + 1] = (float)s;
}

// x[r, off + h * head_stride + 2i .. + 1], i < dims / 2, rotated by the row's table entry
template <typename T>
__global__ void rope_rows_kernel(T* __restrict__ x, int64_t stride, int off, int head_stride, int heads, int dims,
                                 const float* __restrict__ table, int rows) {
    const int half = dims / 2;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)rows * heads * half) return;
    const int k = (int)(i % half);
    const int h = (int)((i / half) % heads);
    const int64_t r = i / ((int64_t)half * heads);
    const float c = table[(r * half + k) * 2], s = table[(r * half + k) * 2 + 1];
    T* p = x + r * stride + off + (int64_t)h * head_stride + 2 * k;
    const float u = to_f32<T>(p[0]), v = to_f32<T>(p[1]);
    p[0] = from_f32<T>(u * c - v * s);
    p[1] = from_f32<T>(v * c + u * s);
}

// One warp per row: src row = [.. | c_raw (kv_rank) at c_off | kr_raw (rot_dim) right behind it].
template <typename T>
__global__ void latent_kv_append_kernel(T* __restrict__ pool, const int32_t* __restrict__ table, int num_slots,
                                        int num_tiles, int total_pages, int tile_size, int kv_rank, int rot_dim,
                                        int rot_dims, const T* __restrict__ src, int64_t src_stride, int c_off,
                                        const float* __restrict__ gain, float eps, const float* __restrict__ rope,
                                        const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                        int rows) {
    const int lane = threadIdx.x & 31;
    const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const int slot = row_slot[r], pos = row_pos[r];
    if (pos < 0 || pos / tile_size >= num_tiles || (unsigned)slot >= (unsigned)num_slots) return;
    const int page = table[(int64_t)slot * num_tiles + pos / tile_size];
    if (page < 0 || page >= total_pages) return;
    const int kd = kv_rank + rot_dim;
    T* dst = pool + ((int64_t)page * tile_size + pos % tile_size) * kd;
    const T* s = src + r * src_stride + c_off;
    float ss = 0.f;
    for (int d = lane; d < kv_rank; d += 32) {
        const float v = to_f32<T>(s[d]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    for (int d = lane; d < kv_rank; d += 32) dst[d] = from_f32<T>(to_f32<T>(s[d]) * rn * gain[d]);
    const int half = rot_dims / 2;
    for (int k = lane; k < half; k += 32) {
        const float c = rope[(r * half + k) * 2], sn = rope[(r * half + k) * 2 + 1];
        const float u = to_f32<T>(s[kv_rank + 2 * k]), v = to_f32<T>(s[kv_rank + 2 * k + 1]);
        dst[kv_rank + 2 * k] = from_f32<T>(u * c - v * sn);
        dst[kv_rank + 2 * k + 1] = from_f32<T>(v * c + u * sn);
    }
    for (int d = rot_dims + lane; d < rot_dim; d += 32) dst[kv_rank + d] = s[kv_rank + d];   // unrotated remainder
}

// RMS norm of `width` columns of strided rows with a per-channel gain (the query latent)
template <typename T>
__global__ void rms_rows_kernel(const T* __restrict__ src, int64_t src_stride, int off, int width, float eps,
                                const float* __restrict__ gain, T* __restrict__ dst, int64_t dst_stride, int rows) {
    const int lane = threadIdx.x & 31;
    const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const T* s = src + r * src_stride + off;
    float ss = 0.f;
    for (int d = lane; d < width; d += 32) {
        const float v = to_f32<T>(s[d]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float rn = 1.0f / sqrtf(ss / (float)width + eps);
    for (int d = lane; d < width; d += 32) dst[r * dst_stride + d] = from_f32<T>(to_f32<T>(s[d]) * rn * gain[d]);
}

// ---- per-head products ----------------------------------------------------------------------------------------------
// out[r * o_rs + h * o_hs + n] = sum_k x[r * x_rs + h * x_hs + k] * W[h][k][n]; CTA = 64 rows x 64 columns of one head.
constexpr int kHlBM = 64, kHlBN = 64, kHlBK = 16;

template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, int64_t x_rs, int64_t x_hs,
                                                          const T* __restrict__ W, int K, int N, int rows,
                                                          T* __restrict__ out, int64_t o_rs, int64_t o_hs) {
    __shared__ float As[kHlBK][kHlBM + 1];
    __shared__ float Bs[kHlBK][kHlBN + 1];
    const int h = blockIdx.z, r0 = blockIdx.x * kHlBM, n0 = blockIdx.y * kHlBN;
    const T* Wh = W + (int64_t)h * K * N;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;   // rows ty * 4 .. + 3, columns tx * 4 .. + 3
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kHlBK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kHlBM * kHlBK; idx += 256) {
            const int r = idx / kHlBK, kk = idx % kHlBK;
            As[kk][r] = (r0 + r < rows && k0 + kk < K) ? to_f32<T>(x[(int64_t)(r0 + r) * x_rs + (int64_t)h * x_hs + k0 + kk]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < kHlBN * kHlBK; idx += 256) {
            const int kk = idx / kHlBN, n = idx % kHlBN;
            Bs[kk][n] = (n0 + n < N && k0 + kk < K) ? to_f32<T>(Wh[(int64_t)(k0 + kk) * N + n0 + n]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kHlBK; ++kk) {
            float av[4], bv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) av[a] = As[kk][ty * 4 + a];
#pragma unroll
            for (int b = 0; b < 4; ++b) bv[b] = Bs[kk][tx * 4 + b];
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int r = r0 + ty * 4 + a;
        if (r >= rows) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int n = n0 + tx * 4 + b;
            if (n < N) out[(int64_t)r * o_rs + (int64_t)h * o_hs + n] = from_f32<T>(acc[a][b]);
        }
    }
}

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ in, int64_t i_rs, int64_t i_hs, const T* __restrict__ gate,
                                 int64_t g_rs, int heads, int vdim, int64_t rows, T* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * heads * vdim) return;
    const int v = (int)(i % vdim), h = (int)((i / vdim) % heads);
    const int64_t r = i / ((int64_t)vdim * heads);
    const float g = sigmoid_f32(to_f32<T>(gate[r * g_rs + h]));
    out[i] = from_f32<T>(to_f32<T>(in[r * i_rs + (int64_t)h * i_hs + v]) * g);
}

// the same on bfloat16 rows with 16-byte aligned head vectors: eight outputs per thread
__global__ void head_gate_bf16x8_kernel(const bf16_t* __restrict__ in, int64_t i_rs, int64_t i_hs, const bf16_t* __restrict__ gate,
                                        int64_t g_rs, int heads, int vdim, int64_t rows, bf16_t* __restrict__ out) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * heads * vdim) return;
    const int v = (int)(i % vdim), h = (int)((i / vdim) % heads);
    const int64_t r = i / ((int64_t)vdim * heads);
    const float g = sigmoid_f32(__bfloat162float(gate[r * g_rs + h]));
    float f[8];
    bf16x8_unpack(*reinterpret_cast<const uint4*>(in + r * i_rs + (int64_t)h * i_hs + v), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] *= g;
    *reinterpret_cast<uint4*>(out + i) = bf16x8_pack(f);
}

// ---- attention: float tile kernel -----------------------------------------------------------------------------------
constexpr int kLaRows = 32;     // (token, head) rows per CTA
constexpr int kLaWarps = 8;
constexpr int kLaRpw = kLaRows / kLaWarps;
constexpr int kLaKeys = 32;     // keys staged per step

struct LatentAttnParams {
    const void* q_lat;          // latent queries: element (row, head, d) at row * ql_rs + head * ql_hs + d, d < kv_rank
    int64_t ql_rs, ql_hs;
    const void* q_rot;          // rotated query parts: (row, head, d) at row * qr_rs + head * qr_hs + d, d < rot_dim
    int64_t qr_rs, qr_hs;
    const void* pool;           // [total_pages][tile_size][kv_rank + rot_dim]
    const int32_t* table;       // [num_slots][num_tiles]
    int num_slots, num_tiles, total_pages, tile_size;
    const int32_t* tiles;       // [ntiles][4]: first row, tokens, slot, position of the first token
    int heads, kv_rank, rot_dim;
    float scale;
    void* out;                  // (row, head, d) at row * o_rs + head * o_hs + d, d < kv_rank
    int64_t o_rs, o_hs;
    int nsplit;
    float* partial;             // nsplit > 1: [(tile, chunk, split, row)][2 + kv_rank], m in natural-log units
    int cta_rows;               // (token, head) rows per CTA: kLaRows (float kernel) or kLmRows (tensor-core kernel)
};

__host__ __device__ __forceinline__ void la_geometry(int heads, int cta_rows, int& hc, int& nchunk) {
    hc = heads < cta_rows ? heads : cta_rows;
    nchunk = (heads + hc - 1) / hc;
}

// A CTA of 8 warps owns up to 32 (token, head) rows: 32 / hc consecutive tokens of one portion x hc = min(32, heads)
// heads; all of them read the same pool rows, staged 32 keys at a time as float (one key per lane for the scores; lanes
// switch to latent columns for the weighted sums, value = the key row's first kv_rank columns).
template <typename T, int NV>
__global__ void __launch_bounds__(kLaWarps * 32) latent_attention_kernel(const LatentAttnParams p) {
    extern __shared__ float smem[];
    const int kd = p.kv_rank + p.rot_dim, kds = kd + 1;
    float* Qs = smem;                              // [32][kd]
    float* Ks = Qs + kLaRows * kd;                 // [32][kd + 1]
    __shared__ int64_t page_row[kLaKeys];

    int hc, nchunk;
    la_geometry(p.heads, kLaRows, hc, nchunk);
    const int bq = kLaRows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1], slot = tile[2], pos0 = tile[3];
    const int chunk = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* pool = static_cast<const T*>(p.pool);

    for (int idx = threadIdx.x; idx < kLaRows * kd; idx += blockDim.x) {
        const int r = idx / kd, d = idx % kd;
        const int tok = r / hc, hh = chunk * hc + r % hc;
        float v = 0.f;
        if (tok < bq && tok < ntok && hh < p.heads) {
            const int64_t row = row0 + tok;
            v = d < p.kv_rank ? to_f32<T>(static_cast<const T*>(p.q_lat)[row * p.ql_rs + hh * p.ql_hs + d])
                              : to_f32<T>(static_cast<const T*>(p.q_rot)[row * p.qr_rs + hh * p.qr_hs + d - p.kv_rank]);
        }
        Qs[idx] = v;
    }

    int rpos[kLaRpw];
    float m[kLaRpw], l[kLaRpw], acc[kLaRpw][NV];
#pragma unroll
    for (int r = 0; r < kLaRpw; ++r) {
        const int row = warp * kLaRpw + r;
        const int tok = row / hc, hh = chunk * hc + row % hc;
        rpos[r] = (tok < bq && tok < ntok && hh < p.heads) ? pos0 + tok : -1;
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[r][i] = 0.f;
    }

    const int total = pos0 + ntok;
    const int nsteps = (total + kLaKeys - 1) / kLaKeys;
    const int per = (nsteps + p.nsplit - 1) / p.nsplit;
    const int s_begin = blockIdx.z * per, s_end = min(nsteps, s_begin + per);

    for (int st = s_begin; st < s_end; ++st) {
        const int c0 = st * kLaKeys;
        __syncthreads();
        if (threadIdx.x < kLaKeys) {
            const int j = c0 + threadIdx.x;
            int64_t pr = -1;
            if (j < total && j / p.tile_size < p.num_tiles) {
                const int page = p.table[(int64_t)slot * p.num_tiles + j / p.tile_size];
                if (page >= 0 && page < p.total_pages) pr = (int64_t)page * p.tile_size + j % p.tile_size;
            }
            page_row[threadIdx.x] = pr;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < kLaKeys * kd; idx += blockDim.x) {
            const int key = idx / kd, d = idx % kd;
            const int64_t pr = page_row[key];
            Ks[key * kds + d] = pr >= 0 ? to_f32<T>(pool[pr * kd + d]) : 0.f;
        }
        __syncthreads();

        float s[kLaRpw];
#pragma unroll
        for (int r = 0; r < kLaRpw; ++r) s[r] = 0.f;
        const float* kr = Ks + lane * kds;
        const float* qb = Qs + warp * kLaRpw * kd;
        for (int d = 0; d < kd; ++d) {
            const float kv = kr[d];
#pragma unroll
            for (int r = 0; r < kLaRpw; ++r) s[r] = fmaf(qb[r * kd + d], kv, s[r]);
        }
        const int j = c0 + lane;
        const bool mapped = page_row[lane] >= 0;
        float pw[kLaRpw];
#pragma unroll
        for (int r = 0; r < kLaRpw; ++r) {
            const bool vis = mapped && j <= rpos[r];
            const float v = vis ? s[r] * p.scale : -INFINITY;
            const float n = fmaxf(m[r], warp_max(v));
            const float c = n == -INFINITY ? 1.f : expf(m[r] - n);
            pw[r] = vis ? expf(v - n) : 0.f;
            l[r] = l[r] * c + warp_sum(pw[r]);
            m[r] = n;
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[r][i] *= c;
        }
        const int nk = min(kLaKeys, total - c0);
        for (int jj = 0; jj < nk; ++jj) {
            float v[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = lane + 32 * i < p.kv_rank ? Ks[jj * kds + lane + 32 * i] : 0.f;
#pragma unroll
            for (int r = 0; r < kLaRpw; ++r) {
                const float w = __shfl_sync(0xffffffffu, pw[r], jj);
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[r][i] = fmaf(w, v[i], acc[r][i]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kLaRpw; ++r) {
        const int row = warp * kLaRpw + r;
        if (p.nsplit > 1) {
            float* dst = p.partial + ((((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit + blockIdx.z) * kLaRows + row) *
                                         (2 + p.kv_rank);
            if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < p.kv_rank) dst[2 + lane + 32 * i] = acc[r][i];
        } else if (rpos[r] >= 0) {
            const int tok = row / hc, hh = chunk * hc + row % hc;
            T* dst = static_cast<T*>(p.out) + (int64_t)(row0 + tok) * p.o_rs + (int64_t)hh * p.o_hs;
            const float inv = 1.0f / l[r];
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < p.kv_rank) dst[lane + 32 * i] = from_f32<T>(acc[r][i] * inv);
        }
    }
}

template <typename T, int NV>
__global__ void __launch_bounds__(kLaWarps * 32) latent_attention_merge_kernel(const LatentAttnParams p) {
    int hc, nchunk;
    la_geometry(p.heads, p.cta_rows, hc, nchunk);
    const int bq = p.cta_rows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1];
    const int chunk = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int row = warp; row < p.cta_rows; row += kLaWarps) {
        const int tok = row / hc, hh = chunk * hc + row % hc;
        if (!(tok < bq && tok < ntok && hh < p.heads)) continue;
        const int64_t zs = (int64_t)p.cta_rows * (2 + p.kv_rank);
        const float* base = p.partial + (((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit * p.cta_rows + row) * (2 + p.kv_rank);
        float M = -INFINITY;
        for (int z = 0; z < p.nsplit; ++z) M = fmaxf(M, base[z * zs]);
        float l = 0.f, acc[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] = 0.f;
        for (int z = 0; z < p.nsplit; ++z) {
            const float* pz = base + z * zs;
            const float w = pz[0] == -INFINITY ? 0.f : expf(pz[0] - M);
            l = fmaf(w, pz[1], l);
#pragma unroll
            for (int i = 0; i < NV; ++i)
                if (lane + 32 * i < p.kv_rank) acc[i] = fmaf(w, pz[2 + lane + 32 * i], acc[i]);
        }
        T* dst = static_cast<T*>(p.out) + (int64_t)(row0 + tok) * p.o_rs + (int64_t)hh * p.o_hs;
        const float inv = 1.0f / l;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (lane + 32 * i < p.kv_rank) dst[lane + 32 * i] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T, int NV>
static int la_launch(const LatentAttnParams& p, int ntiles, cudaStream_t st) {
    const int kd = p.kv_rank + p.rot_dim;
    const size_t smem = ((size_t)kLaRows * kd + (size_t)kLaKeys * (kd + 1)) * sizeof(float);
    if (smem > (size_t)device_info().max_smem_optin) return PA_ERR_UNSUPPORTED;
    auto kern = latent_attention_kernel<T, NV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int hc, nchunk;
    la_geometry(p.heads, kLaRows, hc, nchunk);
    dim3 grid((unsigned)ntiles, (unsigned)nchunk, (unsigned)p.nsplit);
    kern<<<grid, kLaWarps * 32, smem, st>>>(p);
    if (p.nsplit > 1) {
        dim3 g2((unsigned)ntiles, (unsigned)nchunk);
        latent_attention_merge_kernel<T, NV><<<g2, kLaWarps * 32, 0, st>>>(p);
    }
    PA_RETURN_LAUNCH_STATUS();
}

template <typename T>
static int la_dispatch(const LatentAttnParams& p, int ntiles, cudaStream_t st) {
    const int nv = (p.kv_rank + 31) / 32;
    if (nv <= 1) return la_launch<T, 1>(p, ntiles, st);
    if (nv <= 2) return la_launch<T, 2>(p, ntiles, st);
    if (nv <= 4) return la_launch<T, 4>(p, ntiles, st);
    if (nv <= 8) return la_launch<T, 8>(p, ntiles, st);
    if (nv <= 16) return la_launch<T, 16>(p, ntiles, st);
    return PA_ERR_UNSUPPORTED;
}

// ---- attention on the tensor cores (bfloat16) -------------------------------------------------------------------------
// One CTA = up to 64 (token, head) rows that read the same pool rows: 64 / hc consecutive tokens of one portion x hc =
// min(64, heads) heads (a decoded token: its heads alone).  8 warps: warp w owns the 16 rows (w & 3) and the latent
// columns of half (w >> 2) of the output, so the accumulators of a 512-wide latent are 128 registers per thread.  Per
// step 64 keys are located through the page table and brought in with 16-byte cp.async copies into one of two buffers
// (the copies of step t + 1 fly while step t is multiplied); the staged rows serve both products: S = Q K^T over all
// kv_rank + rot_dim columns (mma.sync m16n8k16, bfloat16 operands, float accumulators) and O += P V with V = the first
// kv_rank columns of the same rows, read transposed by ldmatrix.  The two warps of a row group SPLIT the 64 keys of a
// step for the scores (32 each): they exchange their row maxima and then their halves of P (bfloat16, the operand
// type of the second product anyway) through shared memory behind 64-thread named barriers, so no score is computed
// twice; each keeps the sum of its own half and the two sums meet at the end.  A key's validity flag lives in the
// padding of its staged row.  Scores, the running maximum, the exponentials and
// their sum are float; the weights enter the second product rounded to bfloat16, like every other matrix operand of
// this precision.  KVR and ROT are the PADDED sizes: the real kv_rank / rot_dim values (multiples of 8) sit at the start
// of their columns in shared memory, the rest is zero, and 16-wide steps that are all padding are skipped.  nsplit > 1
// cuts the key steps into parts whose (m, l, acc) go to the float kernel's partial layout and merge kernel.
// KSPLIT (decoded tokens of at most 16 heads: every tile is ONE token, so one 16-row group is all the rows there are):
// the four warps of a column half SPLIT the 64 keys of a step, 16 each, over the same rows, and their (m, l, o) meet in
// shared memory at the end -- a quarter of the MMAs per warp, which is what bounds a step that has so few rows.
constexpr int kLmRows = 64, kLmKeys = 64, kLmThreads = 256, kLmPad = 8;

// EXACT: kv_rank == KVR and rot_dim == ROT, so no column is padding and the checks for it fold away.
template <int KVR, int ROT, bool KSPLIT, bool EXACT>
__global__ void __launch_bounds__(kLmThreads, 1) latent_attention_mma_kernel(const LatentAttnParams p) {
    constexpr int KD = KVR + ROT, KS = KD + kLmPad, NT = KVR / 16;     // NT 8-column tiles per warp (half of KVR)
    constexpr int QR = KSPLIT ? 16 : kLmRows;                          // query rows staged
    constexpr int NKG = KSPLIT ? 1 : 2;                                // groups of 16 keys a warp scores per step
    extern __shared__ __align__(16) unsigned char lm_smem[];
    bf16_t* Qs = reinterpret_cast<bf16_t*>(lm_smem);                   // [QR][KS]
    bf16_t* Ks = Qs + QR * KS;                                          // [2][64][KS]; column KD of a row: the key is mapped
    bf16_t* Ps = Ks + 2 * kLmKeys * KS;                                 // !KSPLIT: [4 row groups][16][64] weights

    int hc, nchunk;
    la_geometry(p.heads, kLmRows, hc, nchunk);
    const int bq = kLmRows / hc;
    const int* tile = p.tiles + 4 * blockIdx.x;
    const int row0 = tile[0], ntok = tile[1], slot = tile[2], pos0 = tile[3];
    const int chunk = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp & 3, ch = warp >> 2;
    const int kg0 = KSPLIT ? rg : 2 * ch, rbase = KSPLIT ? 0 : rg * 16;
    bf16_t* Pp = Ps + rg * 16 * kLmKeys;                                // this row group's weights (and its mailbox)
    float* Mb = reinterpret_cast<float*>(Pp);                           // [2 column halves][16 rows], between barriers
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + rg) : "memory"); };
    const int kv_rank = EXACT ? KVR : p.kv_rank, rot_dim = EXACT ? ROT : p.rot_dim, kd = kv_rank + rot_dim;
    const bf16_t* pool = static_cast<const bf16_t*>(p.pool);
    const int32_t* trow = p.table + (int64_t)slot * p.num_tiles;
    const int total = pos0 + ntok;
    const int nkt = (total + kLmKeys - 1) / kLmKeys;
    const int per = (nkt + p.nsplit - 1) / p.nsplit;
    const int kt0 = blockIdx.z * per, kt1 = min(nkt, kt0 + per);

    // queries: piece v of a row is 8 columns of the latent part (v * 8 < KVR) or of the rotated part
    for (int c = tid; c < QR * (KD / 8); c += kLmThreads) {
        const int r = c / (KD / 8), v = c % (KD / 8);
        const int tok = r / hc, hh = chunk * hc + r % hc;
        const bool row_ok = tok < bq && tok < ntok && hh < p.heads;
        const int col = v * 8;
        const bf16_t* src = pool;
        bool ok = false;
        if (row_ok && col < KVR && col < kv_rank) {
            src = static_cast<const bf16_t*>(p.q_lat) + (int64_t)(row0 + tok) * p.ql_rs + (int64_t)hh * p.ql_hs + col;
            ok = true;
        } else if (row_ok && col >= KVR && col - KVR < rot_dim) {
            src = static_cast<const bf16_t*>(p.q_rot) + (int64_t)(row0 + tok) * p.qr_rs + (int64_t)hh * p.qr_hs + col - KVR;
            ok = true;
        }
        cp_async_16(smem_u32(Qs + r * KS + col), src, ok);
    }
    auto pool_row = [&](int j) -> int64_t {
        if (j < total && j / p.tile_size < p.num_tiles) {
            const int page = trow[j / p.tile_size];
            if (page >= 0 && page < p.total_pages) return (int64_t)page * p.tile_size + j % p.tile_size;
        }
        return -1;
    };
    // four threads per key: one page look-up per thread and step, made one step before its copies are issued (the
    // look-up's latency would otherwise sit in front of every step's copies); a thread copies every fourth 16-byte piece
    // of its row
    const int key = tid >> 2, q4 = tid & 3;
    auto load_tile = [&](int64_t pr, int buf) {
        if (q4 == 0) reinterpret_cast<uint16_t*>(Ks + (buf * kLmKeys + key) * KS)[KD] = pr >= 0;
        bf16_t* dst = Ks + (buf * kLmKeys + key) * KS;
        const bf16_t* src = pool + (pr >= 0 ? pr * kd : 0);
#pragma unroll
        for (int i = 0; i < KD / 32; ++i) {
            const int col = (q4 + 4 * i) * 8;
            const bool lat = col < KVR;
            const bool ok = pr >= 0 && (lat ? col < kv_rank : col - KVR < rot_dim);
            cp_async_16(smem_u32(dst + col), ok ? src + (lat ? col : kv_rank + col - KVR) : pool, ok);
        }
    };
    if (kt0 < kt1) load_tile(pool_row(kt0 * kLmKeys + key), 0);
    cp_async_commit();
    int64_t pr_next = kt0 + 1 < kt1 ? pool_row((kt0 + 1) * kLmKeys + key) : -1;

    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[t][c] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int rpos[2];
    bool any_row = false;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rbase + (lane >> 2) + 8 * i;
        const int tok = r / hc, hh = chunk * hc + r % hc;
        rpos[i] = (tok < bq && tok < ntok && hh < p.heads) ? pos0 + tok : -1;
        any_row |= rpos[i] >= 0;
    }
    const bool active = __any_sync(0xffffffffu, any_row);        // this warp has rows with a query
    const float sc = p.scale * 1.4426950408889634f;

    for (int kt = kt0; kt < kt1; ++kt) {
        const int buf = (kt - kt0) & 1, c0 = kt * kLmKeys;
        if (kt + 1 < kt1) load_tile(pr_next, buf ^ 1);
        cp_async_commit();
        pr_next = kt + 2 < kt1 ? pool_row((kt + 2) * kLmKeys + key) : -1;
        cp_async_wait<1>();
        __syncthreads();
        if (active) {
            float s[2 * NKG][4];
#pragma unroll
            for (int t = 0; t < 2 * NKG; ++t)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[t][c] = 0.f;
            // KSPLIT: a warp's two score tiles would be one chain of KD / 16 dependent MMAs each; four sets of
            // accumulators taken in turn cut the chain to a quarter (summed below)
            constexpr int NSET = KSPLIT ? 4 : 1;
            float sx[NSET > 1 ? NSET - 1 : 1][2][4];
            if (KSPLIT) {
#pragma unroll
                for (int e = 0; e < NSET - 1; ++e)
#pragma unroll
                    for (int t = 0; t < 2; ++t)
#pragma unroll
                        for (int c = 0; c < 4; ++c) sx[e][t][c] = 0.f;
            }
#pragma unroll 4
            for (int ks = 0; ks < KD; ks += 16) {
                if (ks < KVR ? ks >= kv_rank : ks - KVR >= rot_dim) continue;      // all padding
                uint32_t a[4];
                ldsm_x4(smem_u32(Qs + (rbase + (lane & 15)) * KS + ks + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
#pragma unroll
                for (int np = 0; np < NKG; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(smem_u32(Ks + (buf * kLmKeys + (kg0 + np) * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + ks + ((lane >> 3) & 1) * 8),
                            b0, b1, b2, b3);
                    const int set = KSPLIT ? (ks / 16) % NSET : 0;
                    if (KSPLIT && set > 0) {
                        mma_bf16_16816(sx[set - 1][0], a, b0, b1);
                        mma_bf16_16816(sx[set - 1][1], a, b2, b3);
                    } else {
                        mma_bf16_16816(s[2 * np], a, b0, b1);
                        mma_bf16_16816(s[2 * np + 1], a, b2, b3);
                    }
                }
            }
            if (KSPLIT) {
#pragma unroll
                for (int e = 0; e < NSET - 1; ++e)
#pragma unroll
                    for (int t = 0; t < 2; ++t)
#pragma unroll
                        for (int c = 0; c < 4; ++c) s[t][c] += sx[e][t][c];
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int t = 0; t < 2 * NKG; ++t) {
                const int col = (2 * kg0 + t) * 8 + 2 * (lane & 3);
                const uint16_t* kok = reinterpret_cast<const uint16_t*>(Ks + (buf * kLmKeys + col) * KS) + KD;
                const int ok0 = kok[0], ok1 = kok[KS];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int i = c >> 1;
                    const bool vis = ((c & 1) ? ok1 : ok0) && c0 + col + (c & 1) <= rpos[i];
                    s[t][c] = vis ? s[t][c] * sc : -INFINITY;
                    mx[i] = fmaxf(mx[i], s[t][c]);
                }
            }
            float ref[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            }
            if (!KSPLIT) {                                       // the row maximum over the partner's 32 keys too
                if ((lane & 3) == 0) {
                    Mb[ch * 16 + (lane >> 2)] = mx[0];
                    Mb[ch * 16 + (lane >> 2) + 8] = mx[1];
                }
                pair_sync();
                mx[0] = fmaxf(mx[0], Mb[(ch ^ 1) * 16 + (lane >> 2)]);
                mx[1] = fmaxf(mx[1], Mb[(ch ^ 1) * 16 + (lane >> 2) + 8]);
                pair_sync();                                     // both have read: the weights may overwrite the mailbox
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
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
            if (!KSPLIT) {                                       // this warp's half of the weights -> shared memory
#pragma unroll
                for (int t = 0; t < 2 * NKG; ++t) {
                    bf16_t* dst = Pp + (lane >> 2) * kLmKeys + (2 * kg0 + t) * 8 + 2 * (lane & 3);
                    *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(s[t][0], s[t][1]);
                    *reinterpret_cast<uint32_t*>(dst + 8 * kLmKeys) = pack_bf16x2(s[t][2], s[t][3]);
                }
                pair_sync();
            }
            constexpr int NPV = KSPLIT ? 1 : 4;                  // groups of 16 keys in the second product
#pragma unroll
            for (int kk = 0; kk < NPV; ++kk) {
                uint32_t a[4];
                if (KSPLIT) {
                    a[0] = pack_bf16x2(s[0][0], s[0][1]);
                    a[1] = pack_bf16x2(s[0][2], s[0][3]);
                    a[2] = pack_bf16x2(s[1][0], s[1][1]);
                    a[3] = pack_bf16x2(s[1][2], s[1][3]);
                } else {
                    ldsm_x4(smem_u32(Pp + (lane & 15) * kLmKeys + kk * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
                }
                const int kg = KSPLIT ? kg0 : kk;
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    const int col0 = ch * (KVR / 2) + np * 16;
                    if (col0 >= kv_rank) continue;               // all padding
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(smem_u32(Ks + (buf * kLmKeys + kg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KS + col0 + (lane >> 4) * 8),
                                  b0, b1, b2, b3);
                    mma_bf16_16816(o[2 * np], a, b0, b1);
                    mma_bf16_16816(o[2 * np + 1], a, b2, b3);
                }
            }
        }
        __syncthreads();                                         // this buffer is free for the copies of step kt + 2
    }
    cp_async_wait<0>();
    bool fin = true;                                             // this warp finishes rows
    if (KSPLIT) {
        // [rg][ch][lane][m0 m1 l0 l1 o...] over the key buffers (odd stride: conflict-free); warp rg == 0 of each column
        // half merges the four parts into its registers
        constexpr int PST = 4 + NT * 4 + 1;
        float* Pm = reinterpret_cast<float*>(Ks);
        float* mine = Pm + ((rg * 2 + ch) * 32 + lane) * PST;
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
                const float* pq = Pm + ((q * 2 + ch) * 32 + lane) * PST;
                M[0] = fmaxf(M[0], pq[0]);
                M[1] = fmaxf(M[1], pq[1]);
            }
            float w0[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                w0[i] = m[i] == -INFINITY ? 0.f : exp2f(m[i] - M[i]);
                l[i] *= w0[i];
                m[i] = M[i];
            }
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[t][c] *= w0[c >> 1];
#pragma unroll
            for (int q = 1; q < 4; ++q) {
                const float* pq = Pm + ((q * 2 + ch) * 32 + lane) * PST;
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
    }
    if (!fin) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    if (!KSPLIT && active) {                                     // the sum over the partner's keys
        if ((lane & 3) == 0) {
            Mb[ch * 16 + (lane >> 2)] = l[0];
            Mb[ch * 16 + (lane >> 2) + 8] = l[1];
        }
        pair_sync();
        l[0] += Mb[(ch ^ 1) * 16 + (lane >> 2)];
        l[1] += Mb[(ch ^ 1) * 16 + (lane >> 2) + 8];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = rbase + (lane >> 2) + 8 * i;
        if (rpos[i] < 0) continue;
        const int tok = r / hc, hh = chunk * hc + r % hc;
        if (p.nsplit > 1) {
            float* dst = p.partial + ((((int64_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit + blockIdx.z) * kLmRows + r) *
                                         (2 + kv_rank);
            if (ch == 0 && (lane & 3) == 0) { dst[0] = m[i] * 0.6931471805599453f; dst[1] = l[i]; }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int col = ch * (KVR / 2) + t * 8 + 2 * (lane & 3);
                if (col < kv_rank) { dst[2 + col] = o[t][2 * i]; dst[2 + col + 1] = o[t][2 * i + 1]; }
            }
        } else {
            const float inv = 1.0f / l[i];
            bf16_t* dst = static_cast<bf16_t*>(p.out) + (int64_t)(row0 + tok) * p.o_rs + (int64_t)hh * p.o_hs;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int col = ch * (KVR / 2) + t * 8 + 2 * (lane & 3);
                if (col < kv_rank) *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16x2(o[t][2 * i] * inv, o[t][2 * i + 1] * inv);
            }
        }
    }
}

template <int NV>
static int lm_merge(const LatentAttnParams& p, int ntiles, int nchunk, cudaStream_t st) {
    latent_attention_merge_kernel<bf16_t, NV><<<dim3((unsigned)ntiles, (unsigned)nchunk), kLaWarps * 32, 0, st>>>(p);
    PA_RETURN_LAUNCH_STATUS();
}

template <int KVR, int ROT, bool KSPLIT>
static int lm_launch_as(const LatentAttnParams& p, int ntiles, cudaStream_t st) {
    const size_t smem = ((size_t)((KSPLIT ? 16 : kLmRows) + 2 * kLmKeys) * (KVR + ROT + kLmPad) + (KSPLIT ? 0 : 4 * 16 * kLmKeys)) *
                        sizeof(bf16_t);
    if (smem > (size_t)device_info().max_smem_optin) return PA_ERR_UNSUPPORTED;
    const bool exact = p.kv_rank == KVR && p.rot_dim == ROT;
    auto kern = exact ? latent_attention_mma_kernel<KVR, ROT, KSPLIT, true> : latent_attention_mma_kernel<KVR, ROT, KSPLIT, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int hc, nchunk;
    la_geometry(p.heads, kLmRows, hc, nchunk);
    kern<<<dim3((unsigned)ntiles, (unsigned)nchunk, (unsigned)p.nsplit), kLmThreads, smem, st>>>(p);
    if (p.nsplit > 1) {
        const int nv = (p.kv_rank + 31) / 32;
        if (nv <= 1) return lm_merge<1>(p, ntiles, nchunk, st);
        if (nv <= 2) return lm_merge<2>(p, ntiles, nchunk, st);
        if (nv <= 4) return lm_merge<4>(p, ntiles, nchunk, st);
        if (nv <= 8) return lm_merge<8>(p, ntiles, nchunk, st);
        return lm_merge<16>(p, ntiles, nchunk, st);
    }
    PA_RETURN_LAUNCH_STATUS();
}

template <int KVR, int ROT>
static int lm_launch(const LatentAttnParams& p, int ntiles, bool one_token_tiles, cudaStream_t st) {
    if (one_token_tiles && p.heads <= 16) return lm_launch_as<KVR, ROT, true>(p, ntiles, st);
    return lm_launch_as<KVR, ROT, false>(p, ntiles, st);
}

static bool lm_shape_ok(int kv_rank, int rot_dim) {
    return kv_rank % 8 == 0 && kv_rank >= 8 && kv_rank <= 512 && rot_dim % 8 == 0 && rot_dim <= 64;
}

// PA_ERR_UNSUPPORTED: this shape or these pointers stay on the float kernel
static int lm_dispatch(const LatentAttnParams& p, int ntiles, bool one_token_tiles, cudaStream_t st) {
    if (!lm_shape_ok(p.kv_rank, p.rot_dim)) return PA_ERR_UNSUPPORTED;
    if (p.ql_rs % 8 || p.ql_hs % 8 || p.o_rs % 2 || p.o_hs % 2) return PA_ERR_UNSUPPORTED;
    if (p.rot_dim && (p.qr_rs % 8 || p.qr_hs % 8 || (uintptr_t)p.q_rot % 16)) return PA_ERR_UNSUPPORTED;
    if ((uintptr_t)p.q_lat % 16 || (uintptr_t)p.pool % 16 || (uintptr_t)p.out % 4) return PA_ERR_UNSUPPORTED;
    const int kp = p.kv_rank <= 64 ? 64 : p.kv_rank <= 128 ? 128 : p.kv_rank <= 256 ? 256 : 512;
    const int rp = p.rot_dim <= 32 ? 32 : 64;
#define PA_LM_CASE(K, R) if (kp == K && rp == R) return lm_launch<K, R>(p, ntiles, one_token_tiles, st)
    PA_LM_CASE(64, 32); PA_LM_CASE(64, 64); PA_LM_CASE(128, 32); PA_LM_CASE(128, 64);
    PA_LM_CASE(256, 32); PA_LM_CASE(256, 64); PA_LM_CASE(512, 32); PA_LM_CASE(512, 64);
#undef PA_LM_CASE
    return PA_ERR_UNSUPPORTED;
}

}  // namespace pa

using namespace pa;

PA_API int pa_rope_table(const int32_t* d_row_pos, int rows, int dims, float base, float* d_table, pa_stream_t stream) {
    PA_CHECK_ARG(d_row_pos && d_table && rows >= 0 && dims >= 0 && dims % 2 == 0 && base > 0.f);
    const int64_t n = (int64_t)rows * (dims / 2);
    if (n == 0) return PA_OK;
    rope_table_kernel<<<(unsigned)((n + 127) / 128), 128, 0, as_stream(stream)>>>(d_row_pos, rows, dims, log((double)base), d_table);
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_rope_rows(void* d_x, int64_t stride, int off, int head_stride, int heads, int dims, const float* d_table,
                        int rows, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_x && d_table && rows >= 0 && heads > 0 && dims >= 0 && dims % 2 == 0);
    const int64_t n = (int64_t)rows * heads * (dims / 2);
    if (n == 0) return PA_OK;
    PA_DISPATCH_ELEM(elem, rope_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<T*>(d_x), stride, off, head_stride, heads, dims, d_table, rows));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_latent_kv_append(void* d_pool, const int32_t* d_table, int num_slots, int num_tiles, int total_pages,
                               int tile_size, int kv_rank, int rot_dim, int rot_dims, const void* d_src, int64_t src_stride,
                               int c_off, const float* d_gain, float eps, const float* d_rope_table,
                               const int32_t* d_row_slot, const int32_t* d_row_pos, int rows, int elem,
                               pa_stream_t stream) {
    PA_CHECK_ARG(d_pool && d_table && d_src && d_gain && d_row_slot && d_row_pos && rows >= 0);
    PA_CHECK_ARG(num_slots > 0 && num_tiles > 0 && total_pages > 0 && tile_size > 0 && kv_rank > 0 && rot_dim >= 0);
    PA_CHECK_ARG(rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 && (rot_dims == 0 || d_rope_table));
    if (rows == 0) return PA_OK;
    const int64_t threads = (int64_t)rows * 32;
    PA_DISPATCH_ELEM(elem, latent_kv_append_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<T*>(d_pool), d_table, num_slots, num_tiles, total_pages, tile_size, kv_rank,
                               rot_dim, rot_dims, static_cast<const T*>(d_src), src_stride, c_off, d_gain, eps,
                               d_rope_table, d_row_slot, d_row_pos, rows));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_rms_norm_rows(const void* d_src, int64_t src_stride, int off, int width, float eps, const float* d_gain,
                            void* d_dst, int64_t dst_stride, int rows, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_src && d_gain && d_dst && width > 0 && rows >= 0);
    if (rows == 0) return PA_OK;
    const int64_t threads = (int64_t)rows * 32;
    PA_DISPATCH_ELEM(elem, rms_rows_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_src), src_stride, off, width, eps, d_gain, static_cast<T*>(d_dst),
                               dst_stride, rows));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_head_linear(const void* d_x, int64_t x_row_stride, int64_t x_head_stride, const void* d_W, int heads, int K,
                          int N, int rows, void* d_out, int64_t o_row_stride, int64_t o_head_stride, int elem,
                          pa_stream_t stream) {
    PA_CHECK_ARG(d_x && d_W && d_out && heads > 0 && K > 0 && N > 0 && rows >= 0);
    if (rows == 0) return PA_OK;
    dim3 grid((unsigned)((rows + kHlBM - 1) / kHlBM), (unsigned)((N + kHlBN - 1) / kHlBN), (unsigned)heads);
    PA_DISPATCH_ELEM(elem, head_linear_kernel<T><<<grid, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_x), x_row_stride, x_head_stride, static_cast<const T*>(d_W), K, N, rows,
                               static_cast<T*>(d_out), o_row_stride, o_head_stride));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_head_gate(const void* d_in, int64_t in_row_stride, int64_t in_head_stride, const void* d_gate,
                        int64_t gate_row_stride, int heads, int vdim, int64_t rows, void* d_out, int elem,
                        pa_stream_t stream) {
    PA_CHECK_ARG(d_in && d_gate && d_out && heads > 0 && vdim > 0 && rows >= 0);
    const int64_t n = rows * heads * vdim;
    if (n == 0) return PA_OK;
    if (elem == 2 && vdim % 8 == 0 && in_row_stride % 8 == 0 && in_head_stride % 8 == 0 && (uintptr_t)d_in % 16 == 0 &&
        (uintptr_t)d_out % 16 == 0) {
        head_gate_bf16x8_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, as_stream(stream)>>>(
            static_cast<const bf16_t*>(d_in), in_row_stride, in_head_stride, static_cast<const bf16_t*>(d_gate), gate_row_stride,
            heads, vdim, rows, static_cast<bf16_t*>(d_out));
        PA_RETURN_LAUNCH_STATUS();
    }
    PA_DISPATCH_ELEM(elem, head_gate_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_in), in_row_stride, in_head_stride, static_cast<const T*>(d_gate),
                               gate_row_stride, heads, vdim, rows, static_cast<T*>(d_out)));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_latent_attention_tile_tokens(int heads) {
    if (heads <= 0) return 0;
    return kLaRows / (heads < kLaRows ? heads : kLaRows);
}

PA_API size_t pa_latent_attention_workspace_bytes(int num_q_tiles, int heads, int kv_rank, int nsplit) {
    if (nsplit <= 1 || num_q_tiles <= 0 || heads <= 0 || kv_rank <= 0) return 0;
    // the larger of the two kernels' geometries (CTA rows x head chunks), so one size serves either tile kind
    size_t most = 0;
    for (int rows : {kLaRows, kLmRows}) {
        int hc, nchunk;
        la_geometry(heads, rows, hc, nchunk);
        const size_t n = (size_t)nchunk * rows;
        most = n > most ? n : most;
    }
    return (size_t)num_q_tiles * nsplit * most * (2 + kv_rank) * sizeof(float);
}

PA_API int pa_latent_attention(const void* d_q_lat, int64_t ql_row_stride, int64_t ql_head_stride, const void* d_q_rot,
                               int64_t qr_row_stride, int64_t qr_head_stride, const void* d_pool, const int32_t* d_table,
                               int num_slots, int num_tiles, int total_pages, int tile_size, const int32_t* d_q_tiles,
                               int num_q_tiles, int heads, int kv_rank, int rot_dim, float scale, void* d_out,
                               int64_t o_row_stride, int64_t o_head_stride, int elem, int nsplit, int tile_kind,
                               void* d_workspace, size_t workspace_bytes, pa_stream_t stream) {
    PA_CHECK_ARG(d_q_lat && (d_q_rot || rot_dim == 0) && d_pool && d_table && d_q_tiles && d_out && num_q_tiles >= 0);
    PA_CHECK_ARG(num_slots > 0 && num_tiles > 0 && total_pages > 0 && tile_size > 0 && heads > 0 && kv_rank > 0 && rot_dim >= 0);
    if (num_q_tiles == 0) return PA_OK;
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 1 && (!d_workspace || workspace_bytes < pa_latent_attention_workspace_bytes(num_q_tiles, heads, kv_rank, nsplit)))
        return PA_ERR_WORKSPACE;
    LatentAttnParams p;
    p.q_lat = d_q_lat; p.ql_rs = ql_row_stride; p.ql_hs = ql_head_stride;
    p.q_rot = d_q_rot; p.qr_rs = qr_row_stride; p.qr_hs = qr_head_stride;
    p.pool = d_pool; p.table = d_table; p.num_slots = num_slots; p.num_tiles = num_tiles; p.total_pages = total_pages;
    p.tile_size = tile_size; p.tiles = d_q_tiles; p.heads = heads; p.kv_rank = kv_rank; p.rot_dim = rot_dim; p.scale = scale;
    p.out = d_out; p.o_rs = o_row_stride; p.o_hs = o_head_stride; p.nsplit = nsplit; p.partial = static_cast<float*>(d_workspace);
    p.cta_rows = tile_kind >= 2 ? kLmRows : kLaRows;
    if (elem != 4 && elem != 2) return PA_ERR_UNSUPPORTED;
    if (tile_kind == 2 || tile_kind == 3)
        return elem == 2 ? lm_dispatch(p, num_q_tiles, tile_kind == 3, as_stream(stream)) : PA_ERR_UNSUPPORTED;
    if (tile_kind != 0) return PA_ERR_UNSUPPORTED;
    if (elem == 4) return la_dispatch<float>(p, num_q_tiles, as_stream(stream));
    return la_dispatch<bf16_t>(p, num_q_tiles, as_stream(stream));
}

PA_API int pa_latent_attention_mma_tile_tokens(int heads, int kv_rank, int rot_dim, int elem) {
    if (heads <= 0 || elem != 2 || !lm_shape_ok(kv_rank, rot_dim)) return 0;
    return kLmRows / (heads < kLmRows ? heads : kLmRows);
}
