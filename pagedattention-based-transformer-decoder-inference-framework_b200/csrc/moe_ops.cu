// moe_ops.cu -- routed feed-forward experts for a batch of token rows.
//
//   router_topk_kernel       float router logits, score function (sigmoid or softmax), the `top` largest per row, optional
//                            renormalisation of the chosen scores, and an optional per-row shared-expert gate
//   moe_sort_kernel          groups the (row, choice) pairs by expert (counting sort) and lists the row tiles of the
//                            grouped matrix products
//   grouped_linear_kernel    out[i] = f(A[src(i)] * s(i)) . W[expert(i)]^T over the sorted pairs, one CTA per
//                            (row tile of one expert, column strip); float accumulation; two epilogues: gate/up pair with
//                            act(gate) * up, or plain rows scattered back to the (row, choice) order as float
//
// Weights are [experts][out][in] in the activation type.  Where the design scales the expert's INPUT by the routing
// weight (instead of its output), `a_scale` carries the weight and the scaled row is rounded to the activation type
// before the product, like any other operand.
#include "seq_common.cuh"

namespace pa {

// ---- router ---------------------------------------------------------------------------------------------------------
// One warp per row.  score_fn: 0 = sigmoid, 1 = softmax over the experts.  Ties go to the lower expert id.
template <typename T>
__global__ void __launch_bounds__(128) router_topk_kernel(const T* __restrict__ h, const float* __restrict__ w_router,
                                                          const float* __restrict__ w_shared_gate, int rows, int width,
                                                          int experts, int top, int score_fn, int renorm,
                                                          int32_t* __restrict__ sel_id, float* __restrict__ sel_w,
                                                          float* __restrict__ shared_gate) {
    extern __shared__ float sc[];                     // [warps][experts]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= rows) return;
    float* s = sc + warp * experts;
    const T* hr = h + (int64_t)row * width;
    for (int e = 0; e < experts; ++e) {
        const float* wr = w_router + (int64_t)e * width;
        float acc = 0.f;
        for (int j = lane; j < width; j += 32) acc = fmaf(to_f32<T>(hr[j]), wr[j], acc);
        acc = warp_sum(acc);
        if (lane == 0) s[e] = acc;
    }
    if (w_shared_gate) {
        float acc = 0.f;
        for (int j = lane; j < width; j += 32) acc = fmaf(to_f32<T>(hr[j]), w_shared_gate[j], acc);
        acc = warp_sum(acc);
        if (lane == 0) shared_gate[row] = sigmoid_f32(acc);
    }
    __syncwarp();
    if (lane == 0) {
        if (score_fn == 0) {
            for (int e = 0; e < experts; ++e) s[e] = sigmoid_f32(s[e]);
        } else {
            float m = -INFINITY, z = 0.f;
            for (int e = 0; e < experts; ++e) m = fmaxf(m, s[e]);
            for (int e = 0; e < experts; ++e) { s[e] = expf(s[e] - m); z += s[e]; }
            for (int e = 0; e < experts; ++e) s[e] /= z;
        }
        float total = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (s[e] > bv) { bv = s[e]; best = e; }
            sel_id[(int64_t)row * top + k] = best;
            sel_w[(int64_t)row * top + k] = bv;
            total += bv;
            s[best] = -INFINITY;
        }
        if (renorm)
            for (int k = 0; k < top; ++k) sel_w[(int64_t)row * top + k] /= total;
    }
}

// ---- grouping -------------------------------------------------------------------------------------------------------
// One CTA.  meta layout (int32): [0, E] exclusive offsets of the experts' pair ranges; then `max_tiles` entries of
// (expert, first sorted pair, pairs) -- expert = -1 marks an unused tile.  order[i] = the (row * top + choice) index of
// sorted pair i.  Pairs of one expert keep no particular order: every output row depends on its own input row only.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t* __restrict__ sel_id, int n, int experts, int tile_rows,
                                                        int max_tiles, int32_t* __restrict__ order,
                                                        int32_t* __restrict__ meta) {
    extern __shared__ int sh[];                       // [experts] counts, [experts + 1] offsets, [experts] cursors
    int* cnt = sh;
    int* off = sh + experts;
    int* cur = off + experts + 1;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel_id[i];
        if (e >= 0 && e < experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, t = 0;
        int32_t* tiles = meta + experts + 1;
        for (int e = 0; e < experts; ++e) {
            off[e] = acc;
            cur[e] = acc;
            meta[e] = acc;
            for (int r = 0; r < cnt[e] && t < max_tiles; r += tile_rows, ++t) {
                tiles[3 * t] = e;
                tiles[3 * t + 1] = acc + r;
                tiles[3 * t + 2] = min(tile_rows, cnt[e] - r);
            }
            acc += cnt[e];
        }
        off[experts] = acc;
        meta[experts] = acc;
        for (; t < max_tiles; ++t) { tiles[3 * t] = -1; tiles[3 * t + 1] = 0; tiles[3 * t + 2] = 0; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sel_id[i];
        if (e >= 0 && e < experts) order[atomicAdd(&cur[e], 1)] = i;
    }
}

// ---- grouped product ------------------------------------------------------------------------------------------------
constexpr int kGlBM = 32, kGlBN = 64, kGlBK = 32;

// MODE 0: A rows gathered from the token rows (order[i] / top), scaled by a_scale[order[i]]; W[e] = [2 * n_out][K]
//         (gate rows, then up rows); out[i][n] = silu(gate) * up in the activation type, sorted order.
// MODE 1: A rows = sorted rows i; W[e] = [n_out][K]; out_f32[order[i]][n] (scatter to the (row, choice) order).
template <typename T, int MODE>
__global__ void __launch_bounds__(256) grouped_linear_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ W,
                                                             int K, int n_out, const int32_t* __restrict__ order,
                                                             const float* __restrict__ a_scale, int top,
                                                             const int32_t* __restrict__ tiles, T* __restrict__ out,
                                                             float* __restrict__ out_f32) {
    __shared__ float As[kGlBK][kGlBM + 1];
    __shared__ float Bs[kGlBK][kGlBN + 1];
    __shared__ float Bu[MODE == 0 ? kGlBK : 1][kGlBN + 1];
    __shared__ int src_row[kGlBM];
    __shared__ float src_scale[kGlBM];
    const int e = tiles[3 * blockIdx.x];
    if (e < 0) return;
    const int i0 = tiles[3 * blockIdx.x + 1], nr = tiles[3 * blockIdx.x + 2];
    const int n0 = blockIdx.y * kGlBN;
    const int w_rows = MODE == 0 ? 2 * n_out : n_out;
    const T* We = W + (int64_t)e * w_rows * K;
    if (threadIdx.x < kGlBM) {
        const int r = threadIdx.x;
        int sr = -1;
        float sc = 1.f;
        if (r < nr) {
            const int pair = order[i0 + r];
            if (MODE == 0) {
                sr = pair / top;
                if (a_scale) sc = a_scale[pair];
            } else {
                sr = i0 + r;
            }
        }
        src_row[r] = sr;
        src_scale[r] = sc;
    }
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;   // rows ty*2 .. +1, columns tx*4 .. +3
    float acc[2][4], accu[2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = accu[a][b] = 0.f;
    for (int k0 = 0; k0 < K; k0 += kGlBK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kGlBM * kGlBK; idx += 256) {
            const int r = idx / kGlBK, kk = idx % kGlBK;
            float v = 0.f;
            const int sr = src_row[r];
            if (sr >= 0 && k0 + kk < K) {
                v = to_f32<T>(A[(int64_t)sr * lda + k0 + kk]);
                if (MODE == 0 && a_scale) v = to_f32<T>(from_f32<T>(v * src_scale[r]));
            }
            As[kk][r] = v;
        }
        for (int idx = threadIdx.x; idx < kGlBN * kGlBK; idx += 256) {
            const int n = idx / kGlBK, kk = idx % kGlBK;
            float v = 0.f, u = 0.f;
            if (n0 + n < n_out && k0 + kk < K) {
                v = to_f32<T>(We[(int64_t)(n0 + n) * K + k0 + kk]);
                if (MODE == 0) u = to_f32<T>(We[(int64_t)(n_out + n0 + n) * K + k0 + kk]);
            }
            Bs[kk][n] = v;
            if (MODE == 0) Bu[kk][n] = u;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kGlBK; ++kk) {
            const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float w = Bs[kk][tx * 4 + b];
                acc[0][b] = fmaf(a0, w, acc[0][b]);
                acc[1][b] = fmaf(a1, w, acc[1][b]);
                if (MODE == 0) {
                    const float u = Bu[kk][tx * 4 + b];
                    accu[0][b] = fmaf(a0, u, accu[0][b]);
                    accu[1][b] = fmaf(a1, u, accu[1][b]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        const int r = ty * 2 + a;
        if (r >= nr) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int n = n0 + tx * 4 + b;
            if (n >= n_out) continue;
            if (MODE == 0) {
                // the two products leave the accumulator in the activation type, like every other projection
                const float gte = to_f32<T>(from_f32<T>(acc[a][b])), up = to_f32<T>(from_f32<T>(accu[a][b]));
                out[(int64_t)(i0 + r) * n_out + n] = from_f32<T>(silu_f32(gte) * up);
            } else {
                out_f32[(int64_t)order[i0 + r] * n_out + n] = acc[a][b];
            }
        }
    }
}

}  // namespace pa

using namespace pa;

PA_API int pa_router_topk(const void* d_h, const float* d_w_router, const float* d_w_shared_gate, int rows, int width,
                          int experts, int top, int score_fn, int renorm, int32_t* d_sel_id, float* d_sel_w,
                          float* d_shared_gate, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_h && d_w_router && d_sel_id && d_sel_w && rows >= 0 && width > 0 && experts > 0);
    PA_CHECK_ARG(top > 0 && top <= experts && (score_fn == 0 || score_fn == 1) && (!d_w_shared_gate || d_shared_gate));
    if (rows == 0) return PA_OK;
    if (experts > 2048) return PA_ERR_UNSUPPORTED;
    const size_t smem = (size_t)4 * experts * sizeof(float);
    PA_DISPATCH_ELEM(elem, router_topk_kernel<T><<<(unsigned)((rows + 3) / 4), 128, smem, as_stream(stream)>>>(
                               static_cast<const T*>(d_h), d_w_router, d_w_shared_gate, rows, width, experts, top,
                               score_fn, renorm, d_sel_id, d_sel_w, d_shared_gate));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_tile_rows(void) { return kGlBM; }

PA_API int pa_moe_max_tiles(int pairs, int experts) {
    return pairs <= 0 || experts <= 0 ? 0 : (pairs + kGlBM - 1) / kGlBM + experts;
}

PA_API size_t pa_moe_meta_ints(int pairs, int experts) {
    return (size_t)experts + 1 + 3 * (size_t)pa_moe_max_tiles(pairs, experts);
}

PA_API int pa_moe_sort(const int32_t* d_sel_id, int pairs, int experts, int32_t* d_order, int32_t* d_meta,
                       pa_stream_t stream) {
    PA_CHECK_ARG(d_sel_id && d_order && d_meta && pairs >= 0 && experts > 0);
    if (pairs == 0) return PA_OK;
    if (experts > 4096) return PA_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(3 * experts + 1) * sizeof(int);
    moe_sort_kernel<<<1, 1024, smem, as_stream(stream)>>>(d_sel_id, pairs, experts, kGlBM, pa_moe_max_tiles(pairs, experts),
                                                         d_order, d_meta);
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_gate_up(const void* d_h, int64_t ldh, const void* d_w_gate_up, int width, int ff, int experts,
                          const int32_t* d_order, const float* d_sel_w, int top, const int32_t* d_meta, int pairs,
                          void* d_act, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_h && d_w_gate_up && d_order && d_meta && d_act && width > 0 && ff > 0 && experts > 0 && top > 0);
    if (pairs <= 0) return PA_OK;
    dim3 grid((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((ff + kGlBN - 1) / kGlBN));
    const int32_t* tiles = d_meta + experts + 1;
    PA_DISPATCH_ELEM(elem, grouped_linear_kernel<T, 0><<<grid, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_h), ldh, static_cast<const T*>(d_w_gate_up), width, ff, d_order,
                               d_sel_w, top, tiles, static_cast<T*>(d_act), nullptr));
    PA_RETURN_LAUNCH_STATUS();
}

PA_API int pa_moe_down(const void* d_act, const void* d_w_down, int ff, int width, int experts, const int32_t* d_order,
                       const int32_t* d_meta, int pairs, float* d_out_pairs, int elem, pa_stream_t stream) {
    PA_CHECK_ARG(d_act && d_w_down && d_order && d_meta && d_out_pairs && width > 0 && ff > 0 && experts > 0);
    if (pairs <= 0) return PA_OK;
    dim3 grid((unsigned)pa_moe_max_tiles(pairs, experts), (unsigned)((width + kGlBN - 1) / kGlBN));
    const int32_t* tiles = d_meta + experts + 1;
    PA_DISPATCH_ELEM(elem, grouped_linear_kernel<T, 1><<<grid, 256, 0, as_stream(stream)>>>(
                               static_cast<const T*>(d_act), (int64_t)ff, static_cast<const T*>(d_w_down), ff, width,
                               d_order, nullptr, 1, tiles, nullptr, d_out_pairs));
    PA_RETURN_LAUNCH_STATUS();
}
