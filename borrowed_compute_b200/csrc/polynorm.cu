// PolyNorm, an activation between the two products of a feed-forward:
//   y = a N(z) + b N(z^2) + c N(z^3) + e
// where powers are taken element by element and N divides a row's vector by its root mean
// square (eps inside the root).  z arrives as float (the product's accumulators, unrounded),
// the three statistics are float sums in a fixed order, and y takes the activation type.
#include "common.cuh"

template <class T>
__global__ void __launch_bounds__(1024) polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, T* __restrict__ out, int F,
                                                       float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];     // weights: written by no kernel
    pdl_wait();
    const float* zr = z + (size_t)blockIdx.x * F;
    T* o = out + (size_t)blockIdx.x * F;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    // A thread's share is taken in ascending order, four at a time where rows are 16-byte aligned.
    if (F % 4 == 0) {
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
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = zr[i], v2 = v * v;
        o[i] = from_f32<T>(fmaf(n1, v, fmaf(n2, v2, fmaf(n3, v2 * v, e))));
    }
}

template <class T> static int launch(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && F > 0, "polynorm: bad sizes rows=%d F=%d", rows, F);
    if (rows == 0) return BC_OK;
    // The block's size depends on the row's width alone, never on the number of rows: a row's sums are the same bits in any batch.
    const int threads = F >= 8192 ? 1024 : F >= 2048 ? 512 : 256;
    bc_launch(polynorm_kernel<T>, dim3(rows), dim3(threads), 0, s, z, coef, (T*)out, F, eps);
    BC_LAUNCH_STATUS();
}
// z: [rows, F] float; coef: the four numbers a, b, c, e; out: [rows, F].
extern "C" int bc_polynorm_f32(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    return launch<float>(z, coef, out, rows, F, eps, s);
}
extern "C" int bc_polynorm_bf16(const float* z, const float* coef, void* out, int rows, int F, float eps, cudaStream_t s) {
    return launch<bf16>(z, coef, out, rows, F, eps, s);
}
