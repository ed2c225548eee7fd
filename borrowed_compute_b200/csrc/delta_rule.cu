// The generalized delta rule: a recurrent mixer whose state is one [D, D] matrix a head
// (key channel i, value channel j) in float, carried from token to token:
//
//   S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T        o_t = S_t^T r_t
//
// with u the key divided by its length, w a decay in (0, 1) and a a removal rate in (0, 1)
// per key channel.  Both corrections read the old state.  Three kernels:
//
//   prepare  (row, head) in parallel: decay, removal rate and unit key from the projections,
//            and the two dot products r.(a*u) and r.k that the output needs;
//   scan     (sequence, head, 32 value channels) walks the rows of the step in time order.
//            A value channel j is independent of the others:
//              s_j' = w * s_j - (a*u) (u . s_j) + k v_j,
//              o_j  = r . s_j' = (r*w) . s_j - (r.(a*u)) (u . s_j) + (r.k) v_j,
//            so one pass over the old column gives both sums.  Eight threads share a column
//            (D/8 key channels each, in registers; two columns a thread, so that every vector it
//            reads from shared memory serves both) and add their sums by shuffles; the
//            step's vectors are staged in shared memory sixteen rows at a time (fewer for wide
//            heads), the next lot copied asynchronously while the current one is walked;
//   finish   (row, head) in parallel: the head's output divided by its root mean square,
//            times a weight, times the sigmoid of a gate.
//
// Everything here is float whatever the activation type is: the projections arrive as float,
// and only the finished output takes the activation type.  What a thread adds and in which
// order depends on the row alone, never on where a prompt was cut or what else is in the batch.
#include "common.cuh"

#define DR_LANES 8          // threads that share one value channel
#define DR_COLS 16          // threads-of-eight a block
#define DR_CJ 2             // value channels a thread: every staged vector it loads serves both
#define DR_BLOCK_COLS (DR_COLS * DR_CJ)
#define DR_MAX_D 256

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// The eight threads that share a value channel hold the key channels in runs of four neighbours, the eight threads'
// runs side by side (a load of 16 bytes a thread then covers 128 bytes without a gap) and the next runs 32 channels
// on: thread `lane` holds channels 32 m + 4 lane .. + 3 for m = 0 .. R/4 - 1.  Heads of at most 16 channels: two
// neighbours a thread.
// The state of one head is stored value channel by value channel: S[j][i], key channel i innermost.
template <int R> __device__ __forceinline__ void load_column(const float* col, int lane, int D, bool ok, float* s) {
    if constexpr (R >= 4) {
#pragma unroll
        for (int m = 0; m < R / 4; m++) {
            const int i = m * 32 + lane * 4;
            if (ok && D % 4 == 0 && i < D) {
                const float4 v = *reinterpret_cast<const float4*>(col + i);
                s[4 * m] = v.x; s[4 * m + 1] = v.y; s[4 * m + 2] = v.z; s[4 * m + 3] = v.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) s[4 * m + e] = ok && i + e < D ? col[i + e] : 0.0f;
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < R; q++) s[q] = ok && lane * R + q < D ? col[lane * R + q] : 0.0f;
    }
}
template <int R> __device__ __forceinline__ void store_column(float* col, int lane, int D, bool ok, const float* s) {
    if (!ok) return;
    if constexpr (R >= 4) {
#pragma unroll
        for (int m = 0; m < R / 4; m++) {
            const int i = m * 32 + lane * 4;
            if (D % 4 == 0 && i < D) {
                *reinterpret_cast<float4*>(col + i) = make_float4(s[4 * m], s[4 * m + 1], s[4 * m + 2], s[4 * m + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (i + e < D) col[i + e] = s[4 * m + e];
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < R; q++)
            if (lane * R + q < D) col[lane * R + q] = s[q];
    }
}
// R values of a staged vector (shared memory, [DP]) in this thread's channel order.
template <int R> __device__ __forceinline__ void load_staged(const float* vec, int lane, float* v) {
    if constexpr (R >= 4) {
#pragma unroll
        for (int m = 0; m < R / 4; m++) {
            const float4 x = *reinterpret_cast<const float4*>(vec + m * 32 + lane * 4);
            v[4 * m] = x.x; v[4 * m + 1] = x.y; v[4 * m + 2] = x.z; v[4 * m + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < R; q++) v[q] = vec[lane * R + q];
    }
}

// proj: [rows, stride] float with r, k, v, gate, a at column offsets 0, HD, 2HD, 3HD, 4HD and the
// decay's inner projection (`inner` wide) at 5HD.  w2t is the decay's outer matrix transposed, [inner, HD], so
// that the threads of a head read neighbouring values.  decay_scale is exp(-1/2) for this rule.  A block takes
// one head of DP_ROWS rows: every value of w2t it reads serves all of them.  Thread d holds channel d of the
// head in every sum, as in the kernels below.
#define DP_ROWS 8
__global__ void delta_prepare_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ w2t, const float* __restrict__ w0,
                                     const float* __restrict__ a_bias, float* __restrict__ decay, float* __restrict__ unit,
                                     float* __restrict__ removal, float* __restrict__ dots, int rows, int H, int D, int inner,
                                     float decay_scale, float key_eps) {
    extern __shared__ float th[];        // tanh of the inner projection, [DP_ROWS][inner]
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int row0 = blockIdx.x * DP_ROWS, head = blockIdx.y, HD = H * D;
    const int n = min(DP_ROWS, rows - row0);
    for (int e = threadIdx.x; e < n * inner; e += blockDim.x) th[e] = tanhf(proj[(size_t)(row0 + e / inner) * stride + 5 * HD + e % inner]);
    __syncthreads();
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    float z[DP_ROWS];
#pragma unroll
    for (int r = 0; r < DP_ROWS; r++) z[r] = 0.0f;
    if (mine) {
#pragma unroll 4
        for (int j = 0; j < inner; j++) {
            const float wv = w2t[(size_t)j * HD + c];
#pragma unroll
            for (int r = 0; r < DP_ROWS; r++) z[r] = fmaf(wv, r < n ? th[r * inner + j] : 0.0f, z[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < DP_ROWS; r++) {
        if (r >= n) break;                       // the same for every thread of the block
        const float* p = proj + (size_t)(row0 + r) * stride;
        float rr = 0.0f, k = 0.0f, a = 0.0f, w = 0.0f;
        if (mine) {
            rr = p[c];
            k = p[HD + c];
            a = sigmoid_f(p[4 * HD + c] + a_bias[c]);
            w = expf(-decay_scale * sigmoid_f(z[r] + w0[c]));
        }
        const float kk = block_sum(k * k, scratch);
        const float u = k / sqrtf(kk + key_eps);
        const float au = a * u;
        const float r_au = block_sum(rr * au, scratch);
        const float r_k = block_sum(rr * k, scratch);
        if (mine) {
            const size_t o = (size_t)(row0 + r) * HD + c;
            decay[o] = w;
            unit[o] = u;
            removal[o] = au;
        }
        if (threadIdx.x == 0) {
            dots[((size_t)(row0 + r) * H + head) * 2] = r_au;
            dots[((size_t)(row0 + r) * H + head) * 2 + 1] = r_k;
        }
    }
}

__device__ __forceinline__ void copy4_async(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The rows of a step are staged DR_STEPS at a time, the next lot on its way (asynchronous copies into the other
// of two buffers) while the current one is walked.
template <int R, int DR_STEPS>   // key channels a thread (D <= 8 R) and rows staged at a time
__global__ void __launch_bounds__(DR_LANES * DR_COLS)
delta_scan_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ decay, const float* __restrict__ unit,
                  const float* __restrict__ removal, const float* __restrict__ dots, float* __restrict__ state,
                  const int* __restrict__ seq_rows, const int* __restrict__ seq_slot, float* __restrict__ out, int H, int D, int n_slots,
                  int write_state) {
    constexpr int DP = DR_LANES * R;
    constexpr int VEC = DR_STEPS * DP;                              // one staged vector: [DR_STEPS][DP]
    constexpr int BUF = 5 * VEC + DR_STEPS * DR_BLOCK_COLS + DR_STEPS * 2;
    __shared__ __align__(16) float sm[2][BUF];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj); PDL_FRESH(decay); PDL_FRESH(unit); PDL_FRESH(removal); PDL_FRESH(dots);
    const int sq = blockIdx.x, head = blockIdx.y, HD = H * D;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    if (slot < 0 || slot >= n_slots || n_new <= 0) return;
    const int lane = threadIdx.x % DR_LANES, col = threadIdx.x / DR_LANES;
    const int j0 = blockIdx.z * DR_BLOCK_COLS + col;                // this thread's value channels: j0 and j0 + DR_COLS
    // Channels past the head's width are never copied to: they stay zero.
    for (int e = threadIdx.x; e < 2 * BUF; e += blockDim.x) (&sm[0][0])[e] = 0.0f;
    __syncthreads();
    auto stage = [&](int t0, int b) {
        const int steps = min(DR_STEPS, n_new - t0);
        float* base = sm[b];
        for (int e = threadIdx.x; e < steps * DP; e += blockDim.x) {
            const int t = e / DP, i = e - t * DP;
            if (i >= D) continue;
            const size_t row = (size_t)(row0 + t0 + t);
            const size_t o = row * HD + (size_t)head * D + i;
            copy4_async(base + e, decay + o);
            copy4_async(base + VEC + e, unit + o);
            copy4_async(base + 2 * VEC + e, removal + o);
            copy4_async(base + 3 * VEC + e, proj + row * stride + (size_t)head * D + i);
            copy4_async(base + 4 * VEC + e, proj + row * stride + HD + (size_t)head * D + i);
        }
        for (int e = threadIdx.x; e < steps * DR_BLOCK_COLS; e += blockDim.x) {
            const int t = e / DR_BLOCK_COLS, cc = e - t * DR_BLOCK_COLS, jj = blockIdx.z * DR_BLOCK_COLS + cc;
            if (jj < D) copy4_async(base + 5 * VEC + e, proj + (size_t)(row0 + t0 + t) * stride + 2 * HD + (size_t)head * D + jj);
        }
        for (int e = threadIdx.x; e < steps * 2; e += blockDim.x)
            copy4_async(base + 5 * VEC + DR_STEPS * DR_BLOCK_COLS + e, dots + ((size_t)(row0 + t0 + e / 2) * H + head) * 2 + e % 2);
    };
    stage(0, 0);
    copies_commit();
    float* S = state + ((size_t)slot * H + head) * D * D;
    float s[DR_CJ][R];
    bool col_ok[DR_CJ];
#pragma unroll
    for (int cj = 0; cj < DR_CJ; cj++) {
        col_ok[cj] = j0 + cj * DR_COLS < D;
        load_column<R>(S + (size_t)(col_ok[cj] ? j0 + cj * DR_COLS : 0) * D, lane, D, col_ok[cj], s[cj]);
    }
    int b = 0;
    for (int t0 = 0; t0 < n_new; t0 += DR_STEPS, b ^= 1) {
        if (t0 + DR_STEPS < n_new) stage(t0 + DR_STEPS, b ^ 1);
        copies_commit();
        copies_wait<1>();
        __syncthreads();
        const int steps = min(DR_STEPS, n_new - t0);
        const float *sw = sm[b], *su = sw + VEC, *sb = su + VEC, *sr = sb + VEC, *sk = sr + VEC, *sv = sk + VEC,
                    *sd = sv + DR_STEPS * DR_BLOCK_COLS;
        for (int t = 0; t < steps; t++) {
            float rws[DR_CJ], us[DR_CJ];
            float vw[R], va[R], vb[R];
            load_staged<R>(sw + t * DP, lane, vw);
            load_staged<R>(sr + t * DP, lane, va);
            load_staged<R>(su + t * DP, lane, vb);
#pragma unroll
            for (int cj = 0; cj < DR_CJ; cj++) {
                rws[cj] = us[cj] = 0.0f;
#pragma unroll
                for (int q = 0; q < R; q++) {
                    rws[cj] = fmaf(va[q] * vw[q], s[cj][q], rws[cj]);
                    us[cj] = fmaf(vb[q], s[cj][q], us[cj]);
                }
            }
#pragma unroll
            for (int o = DR_LANES / 2; o > 0; o >>= 1)
#pragma unroll
                for (int cj = 0; cj < DR_CJ; cj++) {
                    rws[cj] += __shfl_xor_sync(0xffffffffu, rws[cj], o);
                    us[cj] += __shfl_xor_sync(0xffffffffu, us[cj], o);
                }
            load_staged<R>(sk + t * DP, lane, va);
            load_staged<R>(sb + t * DP, lane, vb);
#pragma unroll
            for (int cj = 0; cj < DR_CJ; cj++) {
                const float v = sv[t * DR_BLOCK_COLS + cj * DR_COLS + col];
#pragma unroll
                for (int q = 0; q < R; q++) s[cj][q] = fmaf(va[q], v, fmaf(-vb[q], us[cj], vw[q] * s[cj][q]));
                if (lane == 0 && col_ok[cj])
                    out[(size_t)(row0 + t0 + t) * HD + (size_t)head * D + j0 + cj * DR_COLS] =
                        fmaf(sd[2 * t + 1], v, fmaf(-sd[2 * t], us[cj], rws[cj]));
            }
        }
        __syncthreads();
    }
    copies_wait<0>();
    if (write_state) {
#pragma unroll
        for (int cj = 0; cj < DR_CJ; cj++) store_column<R>(S + (size_t)(col_ok[cj] ? j0 + cj * DR_COLS : 0) * D, lane, D, col_ok[cj], s[cj]);
    }
}

// out[row, c] = o[row, c] / rms(o[row, head(c)]) * weight[c] * sigmoid(gate[row, c]), in the activation type.
// A block takes one head of DP_ROWS rows.
template <class T>
__global__ void delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride, const float* __restrict__ weight,
                                    T* __restrict__ out, int rows, int H, int D, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(o); PDL_FRESH(gate);
    const int row0 = blockIdx.x * DP_ROWS, head = blockIdx.y, HD = H * D;
    const int n = min(DP_ROWS, rows - row0);
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    const float wt = mine ? weight[c] : 0.0f;
    for (int r = 0; r < n; r++) {
        const size_t row = (size_t)(row0 + r);
        const float v = mine ? o[row * HD + c] : 0.0f;
        const float ss = block_sum(v * v, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)D + eps);
        if (mine) out[row * HD + c] = from_f32<T>(v * scale * wt * sigmoid_f(gate[row * gate_stride + c]));
    }
}

// A step of one row a sequence: prepare, one step of the scan and finish in one launch, a block a (row, head)
// with eight threads a value channel.  Every sum is taken by the same threads in the same order as in the three
// kernels above (thread d holds channel d in the sums over a head), so a row decoded alone and the same row in a
// prompt give the same bits.  Heads of up to 128 channels.
template <int R, class T>
__global__ void __launch_bounds__(64 * R)
delta_step_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ w2t, const float* __restrict__ w0,
                  const float* __restrict__ a_bias, const float* __restrict__ norm_w, float* __restrict__ state,
                  const int* __restrict__ row_slot, T* __restrict__ out, int H, int D, int inner, float decay_scale, float key_eps,
                  float norm_eps, int n_slots, int write_state, int slab_in_shared) {
    constexpr int DP = DR_LANES * R;
    extern __shared__ __align__(16) float sm[];
    __shared__ float scratch[32];
    float* th = sm;
    float* sw = th + ((inner + 3) & ~3);      // 16-byte aligned: the dynamic shared memory is, and inner is rounded up to 4
    float *su = sw + DP, *sb = su + DP, *sr = sb + DP, *sk = sr + DP, *so = sk + DP;
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int row = blockIdx.x, head = blockIdx.y, HD = H * D;
    const int slot = row_slot[row];
    if (slot < 0 || slot >= n_slots) return;
    const float* p = proj + (size_t)row * stride;
    for (int j = threadIdx.x; j < inner; j += blockDim.x) th[j] = tanhf(p[5 * HD + j]);
    // The head's slab of the decay matrix, [inner][D], fetched by all threads at once where it fits: the D threads
    // that add it up (in the same order as ever) then read shared memory instead of waiting for one load a term.
    float* slab = so + ((D + 3) & ~3);
    if (slab_in_shared)
        for (int e = threadIdx.x; e < inner * D; e += blockDim.x) slab[e] = w2t[(size_t)(e / D) * HD + head * D + e % D];
    __syncthreads();
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    float r = 0.0f, k = 0.0f, a = 0.0f, w = 0.0f;
    if (mine) {
        r = p[c];
        k = p[HD + c];
        a = sigmoid_f(p[4 * HD + c] + a_bias[c]);
        float z = 0.0f;
        if (slab_in_shared) {
#pragma unroll 8
            for (int j = 0; j < inner; j++) z = fmaf(slab[j * D + d], th[j], z);
        } else {
#pragma unroll 8
            for (int j = 0; j < inner; j++) z = fmaf(w2t[(size_t)j * HD + c], th[j], z);
        }
        w = expf(-decay_scale * sigmoid_f(z + w0[c]));
    }
    const float kk = block_sum(k * k, scratch);
    const float u = k / sqrtf(kk + key_eps);
    const float au = a * u;
    const float r_au = block_sum(r * au, scratch);
    const float r_k = block_sum(r * k, scratch);
    if (d < DP) {
        sw[d] = mine ? w : 0.0f;
        su[d] = mine ? u : 0.0f;
        sb[d] = mine ? au : 0.0f;
        sr[d] = mine ? r : 0.0f;
        sk[d] = mine ? k : 0.0f;
    }
    __syncthreads();
    const int lane = threadIdx.x % DR_LANES, j = threadIdx.x / DR_LANES;
    const bool col_ok = j < D;
    float* S = state + (((size_t)slot * H + head) * D + (col_ok ? j : 0)) * D;      // this thread's column
    float s[R], vw[R], va[R], vb[R];
    load_column<R>(S, lane, D, col_ok, s);
    load_staged<R>(sw, lane, vw);
    load_staged<R>(sr, lane, va);
    load_staged<R>(su, lane, vb);
    float rws = 0.0f, us = 0.0f;
#pragma unroll
    for (int q = 0; q < R; q++) {
        rws = fmaf(va[q] * vw[q], s[q], rws);
        us = fmaf(vb[q], s[q], us);
    }
#pragma unroll
    for (int o = DR_LANES / 2; o > 0; o >>= 1) {
        rws += __shfl_xor_sync(0xffffffffu, rws, o);
        us += __shfl_xor_sync(0xffffffffu, us, o);
    }
    const float v = col_ok ? p[2 * HD + (size_t)head * D + j] : 0.0f;
    if (write_state) {
        load_staged<R>(sk, lane, va);
        load_staged<R>(sb, lane, vb);
#pragma unroll
        for (int q = 0; q < R; q++) s[q] = fmaf(va[q], v, fmaf(-vb[q], us, vw[q] * s[q]));
        store_column<R>(S, lane, D, col_ok, s);
    }
    if (lane == 0 && col_ok) so[j] = fmaf(r_k, v, fmaf(-r_au, us, rws));
    __syncthreads();
    const float o = mine ? so[d] : 0.0f;
    const float ss = block_sum(o * o, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)D + norm_eps);
    if (mine) out[(size_t)row * HD + c] = from_f32<T>(o * scale * norm_w[c] * sigmoid_f(p[3 * HD + c]));
}

template <class T>
static int step(const float* proj, int stride, const float* w2t, const float* w0, const float* a_bias, const float* norm_w, float* state,
                const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale, float key_eps, float norm_eps, int n_slots,
                int write_state, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 128 && inner > 0 && inner <= 1024,
                 "delta_step: bad sizes rows=%d H=%d D=%d inner=%d (a head of at most 128)", rows, H, D, inner);
    BC_CHECK_ARG(stride >= 5 * H * D + inner, "delta_step: a row of %d values cannot hold five projections of %d and %d more", stride, H * D, inner);
    if (rows == 0) return BC_OK;
    const int threads = DR_LANES * ((D + 3) / 4 * 4);
    const dim3 grid(rows, H);
    const size_t slab = (size_t)inner * D * sizeof(float);
    const int slab_in_shared = slab <= 32 * 1024;
#define DS_CASE(R)                                                                                                                      \
    bc_launch(delta_step_kernel<R, T>, grid, dim3(threads),                                                                             \
              (size_t)(((inner + 3) & ~3) + 5 * DR_LANES * R + ((D + 3) & ~3)) * sizeof(float) + (slab_in_shared ? slab : 0), s, proj, \
              stride, w2t, w0, a_bias, norm_w, state, row_slot, (T*)out, H, D, inner, decay_scale, key_eps, norm_eps, n_slots,          \
              write_state, slab_in_shared)
    if (D <= 16) DS_CASE(2);
    else if (D <= 32) DS_CASE(4);
    else if (D <= 64) DS_CASE(8);
    else DS_CASE(16);
#undef DS_CASE
    BC_LAUNCH_STATUS();
}
// One row a sequence (row r lives in slot row_slot[r]; negative: skipped, its row of `out` is left untouched):
// proj as for bc_delta_prepare, state as for bc_delta_scan, out [rows, H D] as from bc_delta_finish.
extern "C" int bc_delta_step_f32(const float* proj, int stride, const float* w2t, const float* w0, const float* a_bias, const float* norm_w,
                                 float* state, const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale,
                                 float key_eps, float norm_eps, int n_slots, int write_state, cudaStream_t s) {
    return step<float>(proj, stride, w2t, w0, a_bias, norm_w, state, row_slot, out, rows, H, D, inner, decay_scale, key_eps, norm_eps, n_slots,
                       write_state, s);
}
extern "C" int bc_delta_step_bf16(const float* proj, int stride, const float* w2t, const float* w0, const float* a_bias, const float* norm_w,
                                  float* state, const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale,
                                  float key_eps, float norm_eps, int n_slots, int write_state, cudaStream_t s) {
    return step<bf16>(proj, stride, w2t, w0, a_bias, norm_w, state, row_slot, out, rows, H, D, inner, decay_scale, key_eps, norm_eps, n_slots,
                      write_state, s);
}

static int threads_for(int D) { return ((D + 31) / 32) * 32; }

extern "C" int bc_delta_prepare(const float* proj, int stride, const float* w2t, const float* w0, const float* a_bias, float* decay, float* unit,
                                float* removal, float* dots, int rows, int H, int D, int inner, float decay_scale, float key_eps,
                                cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 1024 && inner > 0 && inner <= 1024,
                 "delta_prepare: bad sizes rows=%d H=%d D=%d inner=%d (an inner width of at most 1024)", rows, H, D, inner);
    BC_CHECK_ARG(stride >= 5 * H * D + inner, "delta_prepare: a row of %d values cannot hold five projections of %d and %d more", stride, H * D, inner);
    if (rows == 0) return BC_OK;
    bc_launch(delta_prepare_kernel, dim3((rows + DP_ROWS - 1) / DP_ROWS, H), dim3(threads_for(D)), (size_t)DP_ROWS * inner * sizeof(float), s, proj,
              stride, w2t, w0, a_bias, decay, unit, removal, dots, rows, H, D, inner, decay_scale, key_eps);
    BC_LAUNCH_STATUS();
}

// state: [n_slots, H, D, D] float, value channel before key channel.  Sequence s owns rows seq_rows[s] .. seq_rows[s + 1] and lives in
// slot seq_slot[s] (negative: skipped, its rows of `out` are left untouched).  write_state 0 leaves
// the state as it was.
extern "C" int bc_delta_scan(const float* proj, int stride, const float* decay, const float* unit, const float* removal, const float* dots,
                             float* state, const int* seq_rows, const int* seq_slot, float* out, int seqs, int H, int D, int n_slots,
                             int write_state, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 2147483647 && H > 0 && H <= 65535 && D > 0 && D <= DR_MAX_D,
                 "delta_scan: bad sizes seqs=%d H=%d D=%d (a head of at most %d)", seqs, H, D, DR_MAX_D);
    if (seqs == 0) return BC_OK;
    const dim3 grid(seqs, H, (D + DR_BLOCK_COLS - 1) / DR_BLOCK_COLS), block(DR_LANES * DR_COLS);
#define DR_CASE(R, STEPS)                                                                                                                      \
    bc_launch(delta_scan_kernel<R, STEPS>, grid, block, 0, s, proj, stride, decay, unit, removal, dots, state, seq_rows, seq_slot, out, H, D, \
              n_slots, write_state)
    if (D <= 16) DR_CASE(2, 16);
    else if (D <= 32) DR_CASE(4, 16);
    else if (D <= 64) DR_CASE(8, 16);
    else if (D <= 128) DR_CASE(16, 8);
    else DR_CASE(32, 4);      // 64 state values a thread
#undef DR_CASE
    BC_LAUNCH_STATUS();
}

template <class T>
static int finish(const float* o, const float* gate, int gate_stride, const float* weight, void* out, int rows, int H, int D, float eps,
                  cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 1024, "delta_finish: bad sizes rows=%d H=%d D=%d", rows, H, D);
    if (rows == 0) return BC_OK;
    bc_launch(delta_finish_kernel<T>, dim3((rows + DP_ROWS - 1) / DP_ROWS, H), dim3(threads_for(D)), 0, s, o, gate, gate_stride, weight, (T*)out,
              rows, H, D, eps);
    BC_LAUNCH_STATUS();
}
extern "C" int bc_delta_finish_f32(const float* o, const float* gate, int gate_stride, const float* weight, void* out, int rows, int H, int D,
                                   float eps, cudaStream_t s) {
    return finish<float>(o, gate, gate_stride, weight, out, rows, H, D, eps, s);
}
extern "C" int bc_delta_finish_bf16(const float* o, const float* gate, int gate_stride, const float* weight, void* out, int rows, int H, int D,
                                    float eps, cudaStream_t s) {
    return finish<bf16>(o, gate, gate_stride, weight, out, rows, H, D, eps, s);
}
