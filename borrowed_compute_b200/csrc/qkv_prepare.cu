// What lies between the fused q/k/v product and attention when queries and keys are
// normalised as wholes: for every row
//   q, k, v  += their biases (if any)
//   q, k      = RMS norm over the whole projection (all heads at once), times a weight
//   q, k      rotated by the row's position on the first `rot` dimensions of each head,
//             dimension i paired with i + rot/2 (the rest pass unchanged)
//   q        -> the activation type, for the attention kernel
//   k, v     -> the row's place in the paged cache (planes of different widths D and DV)
// The projection arrives as float (the product's accumulators); statistics, angles and the
// rotation are float.  One block a row.
#include "common.cuh"

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
template <class T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// WIDE: every width (heads' sizes, half the rotated dimensions) is a multiple of 4, so a thread takes four
// neighbouring values at a time, which lie in one head and on one side of the rotation.  Else one at a time.
// Which values a thread adds up, and in which order, depends on the sizes alone.
template <class T, bool WIDE>
__global__ void __launch_bounds__(1024)
qkv_prepare_kernel(const float* __restrict__ qkv, const float* __restrict__ bias, const float* __restrict__ q_weight,
                   const float* __restrict__ k_weight, const float* __restrict__ cos_sin, int n_positions, const int* __restrict__ row_pos,
                   const int* __restrict__ row_slot, const int* __restrict__ page_table, int max_pages, int n_pages, T* __restrict__ q_out,
                   T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G, int D, int DV, int rot, float eps, int normed,
                   int write_cache) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(qkv);
    const int r = blockIdx.x;
    const int nq = H * D, nk = G * D, nv = G * DV;
    const float* x = qkv + (size_t)r * (nq + nk + nv);
    const int slot = row_slot[r];
    const int pos = row_pos[r];
    float q_scale = 1.0f, k_scale = 1.0f;
    if (normed) {
        float sq = 0.0f, sk = 0.0f;
        if (WIDE) {
            for (int i = 4 * threadIdx.x; i < nq + nk; i += 4 * blockDim.x) {
                float4 v = *reinterpret_cast<const float4*>(x + i);
                if (bias) v = add4(v, *reinterpret_cast<const float4*>(bias + i));
                const float s = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, v.x * v.x)));
                if (i < nq) sq += s; else sk += s;
            }
        } else {
            for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
                const float v = x[i] + (bias ? bias[i] : 0.0f);
                if (i < nq) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
            }
        }
        q_scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
        k_scale = 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps);
    }
    const int half = rot / 2;
    const bool turn = rot > 0 && cos_sin != nullptr && pos >= 0 && pos < n_positions;
    const float* cs = cos_sin + (size_t)(turn ? pos : 0) * half * 2;
    int page = -1;
    if (slot >= 0 && pos >= 0 && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    if (page >= n_pages) page = -1;
    const bool cache = write_cache && page >= 0;
    // Queries and keys are one loop: element i < nq is a query, the others keys.
    if (WIDE) {
        for (int i = 4 * threadIdx.x; i < nq + nk; i += 4 * blockDim.x) {
            const bool is_q = i < nq;
            const int e = is_q ? i : i - nq;
            const int head = e / D, d = e - head * D;
            const float scale = is_q ? q_scale : k_scale;
            const float* wt = is_q ? q_weight : k_weight;
            float4 v = *reinterpret_cast<const float4*>(x + i);
            if (bias) v = add4(v, *reinterpret_cast<const float4*>(bias + i));
            float4 w4 = make_float4(scale, scale, scale, scale);
            if (normed) {
                const float4 g = *reinterpret_cast<const float4*>(wt + e);
                w4 = make_float4(scale * g.x, scale * g.y, scale * g.z, scale * g.w);
            }
            v = make_float4(v.x * w4.x, v.y * w4.y, v.z * w4.z, v.w * w4.w);
            if (turn && d < rot) {
                const int other = d < half ? i + half : i - half, eo = d < half ? e + half : e - half;
                float4 p = *reinterpret_cast<const float4*>(x + other);
                if (bias) p = add4(p, *reinterpret_cast<const float4*>(bias + other));
                float4 pw = make_float4(scale, scale, scale, scale);
                if (normed) {
                    const float4 g = *reinterpret_cast<const float4*>(wt + eo);
                    pw = make_float4(scale * g.x, scale * g.y, scale * g.z, scale * g.w);
                }
                p = make_float4(p.x * pw.x, p.y * pw.y, p.z * pw.z, p.w * pw.w);
                const int pair = d < half ? d : d - half;
                const float4 c0 = *reinterpret_cast<const float4*>(cs + 2 * pair), c1 = *reinterpret_cast<const float4*>(cs + 2 * pair + 4);
                // (cos, sin) of the four pairs: c0 = (c, s, c, s), c1 = (c, s, c, s)
                if (d < half) v = make_float4(v.x * c0.x - p.x * c0.y, v.y * c0.z - p.y * c0.w, v.z * c1.x - p.z * c1.y, v.w * c1.z - p.w * c1.w);
                else v = make_float4(v.x * c0.x + p.x * c0.y, v.y * c0.z + p.y * c0.w, v.z * c1.x + p.z * c1.y, v.w * c1.z + p.w * c1.w);
            }
            if (is_q) store4<T>(q_out + (size_t)r * nq + e, v);
            else if (cache) store4<T>(k_cache + (((size_t)page * G + head) * BC_PAGE + pos % BC_PAGE) * D + d, v);
        }
        if (cache) {
            for (int i = 4 * threadIdx.x; i < nv; i += 4 * blockDim.x) {
                const int g = i / DV, d = i - g * DV;
                float4 v = *reinterpret_cast<const float4*>(x + nq + nk + i);
                if (bias) v = add4(v, *reinterpret_cast<const float4*>(bias + nq + nk + i));
                store4<T>(v_cache + (((size_t)page * G + g) * BC_PAGE + pos % BC_PAGE) * DV + d, v);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const bool is_q = i < nq;
        const int e = is_q ? i : i - nq;
        const int d = e % D;
        const float scale = is_q ? q_scale : k_scale;
        const float* wt = is_q ? q_weight : k_weight;
        float v = (x[i] + (bias ? bias[i] : 0.0f)) * (normed ? scale * wt[e] : scale);
        if (turn && d < rot) {
            const int other = d < half ? i + half : i - half, eo = d < half ? e + half : e - half;
            const float p = (x[other] + (bias ? bias[other] : 0.0f)) * (normed ? scale * wt[eo] : scale);
            const float c = cs[2 * (d % half)], s = cs[2 * (d % half) + 1];
            v = d < half ? v * c - p * s : v * c + p * s;
        }
        if (is_q) {
            q_out[(size_t)r * nq + e] = from_f32<T>(v);
        } else if (cache) {
            const int g = e / D;
            k_cache[(((size_t)page * G + g) * BC_PAGE + pos % BC_PAGE) * D + d] = from_f32<T>(v);
        }
    }
    if (cache) {
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            const int g = i / DV, d = i % DV;
            v_cache[(((size_t)page * G + g) * BC_PAGE + pos % BC_PAGE) * DV + d] = from_f32<T>(x[nq + nk + i] + (bias ? bias[nq + nk + i] : 0.0f));
        }
    }
}

template <class T>
static int launch(const float* qkv, const float* bias, const float* q_weight, const float* k_weight, const float* cos_sin, int n_positions,
                  const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out, void* k_cache,
                  void* v_cache, int rows, int H, int G, int D, int DV, int rot, float eps, int normed, int write_cache, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && D > 0 && DV > 0, "qkv_prepare: bad sizes rows=%d H=%d G=%d D=%d DV=%d", rows, H, G, D, DV);
    BC_CHECK_ARG(rot >= 0 && rot % 2 == 0 && rot <= D, "qkv_prepare: %d rotated dimensions of a head of %d", rot, D);
    BC_CHECK_ARG(!normed || (q_weight && k_weight), "qkv_prepare: the norm needs its weights");
    if (rows == 0) return BC_OK;
    // The block's size depends on the row's width alone, never on the number of rows: a row's sums are the same bits in any batch.
    const int width = H * D + G * D;
    const int threads = width >= 8192 ? 1024 : width >= 2048 ? 512 : 256;
    // Four values at a time where every width is a multiple of 4 (half the rotated dimensions too: the table's rows are then
    // 16-byte aligned pairs of pairs) and every pointer is 16-byte aligned.
    const bool wide = D % 4 == 0 && DV % 4 == 0 && rot % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)bias % 16 == 0 &&
                      (uintptr_t)q_weight % 16 == 0 && (uintptr_t)k_weight % 16 == 0 && (uintptr_t)cos_sin % 16 == 0 &&
                      (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0;
    if (wide)
        bc_launch(qkv_prepare_kernel<T, true>, dim3(rows), dim3(threads), 0, s, qkv, bias, q_weight, k_weight, cos_sin, n_positions, row_pos,
                  row_slot, page_table, max_pages, n_pages, (T*)q_out, (T*)k_cache, (T*)v_cache, H, G, D, DV, rot, eps, normed, write_cache);
    else
        bc_launch(qkv_prepare_kernel<T, false>, dim3(rows), dim3(threads), 0, s, qkv, bias, q_weight, k_weight, cos_sin, n_positions, row_pos,
                  row_slot, page_table, max_pages, n_pages, (T*)q_out, (T*)k_cache, (T*)v_cache, H, G, D, DV, rot, eps, normed, write_cache);
    BC_LAUNCH_STATUS();
}

// qkv: [rows, H D + G D + G DV] float; bias: the same width or null; q_weight [H D], k_weight [G D]
// (used when normed); cos_sin: [n_positions, rot / 2, 2] or null; q_out: [rows, H D];
// k_cache [pages, G, PAGE, D], v_cache [pages, G, PAGE, DV].  Rows whose slot is negative
// write no cache.
extern "C" int bc_qkv_prepare_f32(const float* qkv, const float* bias, const float* q_weight, const float* k_weight, const float* cos_sin,
                                  int n_positions, const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages,
                                  void* q_out, void* k_cache, void* v_cache, int rows, int H, int G, int D, int DV, int rot, float eps,
                                  int normed, int write_cache, cudaStream_t s) {
    return launch<float>(qkv, bias, q_weight, k_weight, cos_sin, n_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache,
                         v_cache, rows, H, G, D, DV, rot, eps, normed, write_cache, s);
}
extern "C" int bc_qkv_prepare_bf16(const float* qkv, const float* bias, const float* q_weight, const float* k_weight, const float* cos_sin,
                                   int n_positions, const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages,
                                   void* q_out, void* k_cache, void* v_cache, int rows, int H, int G, int D, int DV, int rot, float eps,
                                   int normed, int write_cache, cudaStream_t s) {
    return launch<bf16>(qkv, bias, q_weight, k_weight, cos_sin, n_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache,
                        v_cache, rows, H, G, D, DV, rot, eps, normed, write_cache, s);
}

// ------------------------------------------------------------------------ norm a head
// The same place in a layer for models that normalise every head of q and of k by itself: an RMS norm over
// the head's D values with one weight of D values that all heads share (separately for q and for k), then
// the rotation of the first `rot` dimensions, then q to the activation type and k, v into the cache.
// `pairing` 0 pairs dimension i with i + rot/2, 1 pairs 2i with 2i + 1.  One warp a (row, head): the lanes
// take pairs of dimensions, so the sum of squares and the rotation need no second pass over memory; which
// values a lane adds, and in which order, depends on the sizes alone.
template <class T>
__global__ void __launch_bounds__(256)
qkv_prepare_heads_kernel(const float* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                         const float* __restrict__ cos_sin, int n_positions, const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                         const int* __restrict__ page_table, int max_pages, int n_pages, T* __restrict__ q_out, T* __restrict__ k_cache,
                         T* __restrict__ v_cache, int H, int G, int D, int DV, int rot, int pairing, float eps, int normed, int write_cache) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(qkv);
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int nq = H * D, nk = G * D, nv = G * DV;
    const float* x = qkv + (size_t)r * (nq + nk + nv);
    const int slot = row_slot[r];
    const int pos = row_pos[r];
    const int half = rot / 2;
    const bool turn = rot > 0 && cos_sin != nullptr && pos >= 0 && pos < n_positions;
    const float* cs = cos_sin + (size_t)(turn ? pos : 0) * half * 2;
    int page = -1;
    if (slot >= 0 && pos >= 0 && pos / BC_PAGE < max_pages) page = page_table[(size_t)slot * max_pages + pos / BC_PAGE];
    if (page >= n_pages) page = -1;
    const bool cache = write_cache && page >= 0;
    const int units = half + (D - rot);          // pairs that turn, then single dimensions that pass
    for (int head = warp; head < H + G; head += warps) {
        const bool is_q = head < H;
        const float* xh = x + (size_t)head * D;      // keys follow the queries in the projection
        const float* wt = is_q ? q_weight : k_weight;
        float ss = 0.0f;
        if (normed) {
            for (int d = lane; d < D; d += 32) ss = fmaf(xh[d], xh[d], ss);
            ss = warp_sum(ss);
        }
        const float scale = normed ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
        T* dst = is_q ? q_out + (size_t)r * nq + (size_t)head * D
                      : k_cache + (((size_t)(cache ? page : 0) * G + (head - H)) * BC_PAGE + pos % BC_PAGE) * D;
        if (!is_q && !cache) continue;
        for (int u = lane; u < units; u += 32) {
            if (u < half) {
                const int a = pairing ? 2 * u : u, b = pairing ? 2 * u + 1 : u + half;
                float va = xh[a] * (normed ? scale * wt[a] : 1.0f), vb = xh[b] * (normed ? scale * wt[b] : 1.0f);
                if (turn) {
                    const float c = cs[2 * u], s = cs[2 * u + 1];
                    const float ra = va * c - vb * s, rb = vb * c + va * s;
                    va = ra;
                    vb = rb;
                }
                dst[a] = from_f32<T>(va);
                dst[b] = from_f32<T>(vb);
            } else {
                const int d = rot + (u - half);
                dst[d] = from_f32<T>(xh[d] * (normed ? scale * wt[d] : 1.0f));
            }
        }
    }
    if (cache) {
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            const int g = i / DV, d = i - g * DV;
            v_cache[(((size_t)page * G + g) * BC_PAGE + pos % BC_PAGE) * DV + d] = from_f32<T>(x[nq + nk + i]);
        }
    }
}

template <class T>
static int launch_heads(const float* qkv, const float* q_weight, const float* k_weight, const float* cos_sin, int n_positions, const int* row_pos,
                        const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out, void* k_cache, void* v_cache, int rows,
                        int H, int G, int D, int DV, int rot, int pairing, float eps, int normed, int write_cache, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && G > 0 && D > 0 && DV > 0, "qkv_prepare_heads: bad sizes rows=%d H=%d G=%d D=%d DV=%d", rows, H, G, D, DV);
    BC_CHECK_ARG(rot >= 0 && rot % 2 == 0 && rot <= D, "qkv_prepare_heads: %d rotated dimensions of a head of %d", rot, D);
    BC_CHECK_ARG(!normed || (q_weight && k_weight), "qkv_prepare_heads: the norm needs its weights");
    if (rows == 0) return BC_OK;
    const int heads = H + G;
    const int threads = heads >= 8 ? 256 : heads >= 4 ? 128 : 64;      // by the row's heads alone
    bc_launch(qkv_prepare_heads_kernel<T>, dim3(rows), dim3(threads), 0, s, qkv, q_weight, k_weight, cos_sin, n_positions, row_pos, row_slot,
              page_table, max_pages, n_pages, (T*)q_out, (T*)k_cache, (T*)v_cache, H, G, D, DV, rot, pairing, eps, normed, write_cache);
    BC_LAUNCH_STATUS();
}

// As bc_qkv_prepare_*, without biases; q_weight and k_weight hold D values each; cos_sin: [n_positions, rot / 2, 2].
extern "C" int bc_qkv_prepare_heads_f32(const float* qkv, const float* q_weight, const float* k_weight, const float* cos_sin, int n_positions,
                                        const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out,
                                        void* k_cache, void* v_cache, int rows, int H, int G, int D, int DV, int rot, int pairing, float eps,
                                        int normed, int write_cache, cudaStream_t s) {
    return launch_heads<float>(qkv, q_weight, k_weight, cos_sin, n_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache,
                               v_cache, rows, H, G, D, DV, rot, pairing, eps, normed, write_cache, s);
}
extern "C" int bc_qkv_prepare_heads_bf16(const float* qkv, const float* q_weight, const float* k_weight, const float* cos_sin, int n_positions,
                                         const int* row_pos, const int* row_slot, const int* page_table, int max_pages, int n_pages, void* q_out,
                                         void* k_cache, void* v_cache, int rows, int H, int G, int D, int DV, int rot, int pairing, float eps,
                                         int normed, int write_cache, cudaStream_t s) {
    return launch_heads<bf16>(qkv, q_weight, k_weight, cos_sin, n_positions, row_pos, row_slot, page_table, max_pages, n_pages, q_out, k_cache,
                              v_cache, rows, H, G, D, DV, rot, pairing, eps, normed, write_cache, s);
}
