// PolyNorm, an activation between the two products of a feed-forward:
//   y = a N(z) + b N(z^2) + c N(z^3) + e
// where powers are taken element by element and N divides a row's vector by its root mean
// square (eps inside the root).  z arrives as float (the product's accumulators, unrounded),
// the three statistics are float sums in a fixed order, and y takes the activation type.
#include "common.cuh"

template <class T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// KEEP > 0: rows of at most 4 KEEP values a thread (and a multiple of 4 wide) stay in registers between the two passes, so
// a row is read once.
template <class T, int KEEP>
__global__ void __launch_bounds__(1024) polynorm_kernel(const float* z, const float* __restrict__ coef, T* out, int F, float eps) {
    // z and out are deliberately not __restrict__: z is what the kernel before wrote, and a pointer the compiler may take
    // for never-written memory lets it move the loads of a kept row above pdl_wait() (seen: wrong rows inside a model,
    // right ones when the kernel ran alone).
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];     // weights: written by no kernel
    pdl_wait();
    PDL_FRESH(z);
    const float* zr = z + (size_t)blockIdx.x * F;
    T* o = out + (size_t)blockIdx.x * F;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    // A thread's share is taken in ascending order, four at a time where rows are 16-byte aligned.
    float4 kept[KEEP > 0 ? KEEP : 1];
    if (KEEP > 0) {
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = 4 * (threadIdx.x + j * blockDim.x);
            kept[j] = i < F ? *reinterpret_cast<const float4*>(zr + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            if (4 * (threadIdx.x + j * blockDim.x) >= F) break;
            const float e4[4] = {kept[j].x, kept[j].y, kept[j].z, kept[j].w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float v = e4[k], v2 = v * v;
                s1 += v2;
                s2 = fmaf(v2, v2, s2);
                s3 = fmaf(v2 * v, v2 * v, s3);
            }
        }
    } else if (F % 4 == 0) {
        for (int i = 4 * threadIdx.x; i < F; i += 4 * blockDim.x) {
            const float4 q = *reinterpret_cast<const float4*>(zr + i);
            const float e4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float v = e4[k], v2 = v * v;
                s1 += v2;
                s2 = fmaf(v2, v2, s2);
                s3 = fmaf(v2 * v, v2 * v, s3);
            }
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) {
            const float v = zr[i], v2 = v * v;
            s1 += v2;
            s2 = fmaf(v2, v2, s2);
            s3 = fmaf(v2 * v, v2 * v, s3);
        }
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float n1 = a / sqrtf(s1 / (float)F + eps), n2 = b / sqrtf(s2 / (float)F + eps), n3 = c / sqrtf(s3 / (float)F + eps);
    auto act = [&](float v) { const float v2 = v * v; return fmaf(n1, v, fmaf(n2, v2, fmaf(n3, v2 * v, e))); };
    if (KEEP > 0) {
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            const int i = 4 * (threadIdx.x + j * blockDim.x);
            if (i < F) store4<T>(o + i, make_float4(act(kept[j].x), act(kept[j].y), act(kept[j].z), act(kept[j].w)));
        }
    } else if (F % 4 == 0) {
        for (int i = 4 * threadIdx.x; i < F; i += 4 * blockDim.x) {
            const float4 q = *reinterpret_cast<const float4*>(zr + i);
            store4<T>(o + i, make_float4(act(q.x), act(q.y), act(q.z), act(q.w)));
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) o[i] = from_f32<T>(act(zr[i]));
    }
}

static int g_polynorm_mode = 0;      // measurements: 1 keeps no row in registers (two passes over memory)
extern "C" void bc_polynorm_set_mode(int m) { g_polynorm_mode = m; }

template <class T> static int launch(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && F > 0, "polynorm: bad sizes rows=%d F=%d", rows, F);
    if (rows == 0) return BC_OK;
    // The block's size depends on the row's width alone, never on the number of rows: a row's sums are the same bits in any batch.
    // Small blocks that keep their row (eight vectors of four a thread) put several rows on an SM at different points of
    // their lives: 2,048 rows of 14,336 took 60 us with 1,024 threads a row (one block an SM by its registers), 44 us with 512.
    const int threads = F <= 8192 ? 256 : F <= 16384 ? 512 : 1024;
    const bool keep = g_polynorm_mode != 1 && F % 4 == 0 && F <= 32 * threads;
    if (keep)
        bc_launch(polynorm_kernel<T, 8>, dim3(rows), dim3(threads), 0, s, z, coef, (T*)out, F, eps);
    else
        bc_launch(polynorm_kernel<T, 0>, dim3(rows), dim3(threads), 0, s, z, coef, (T*)out, F, eps);
    BC_LAUNCH_STATUS();
}
// z: [rows, F] float; coef: the four numbers a, b, c, e; out: [rows, F].
extern "C" int bc_polynorm_f32(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    return launch<float>(z, coef, out, rows, F, eps, s);
}
extern "C" int bc_polynorm_bf16(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    return launch<bf16>(z, coef, out, rows, F, eps, s);
}
