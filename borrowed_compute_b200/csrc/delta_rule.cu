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
//   scan     (sequence, head, 16 value channels) walks the rows of the step in time order.
//            A value channel j is independent of the others:
//              s_j' = w * s_j - (a*u) (u . s_j) + k v_j,
//              o_j  = r . s_j' = (r*w) . s_j - (r.(a*u)) (u . s_j) + (r.k) v_j,
//            so one pass over the old column gives both sums.  Eight threads share a column
//            (D/8 key channels each, in registers) and add their sums by shuffles; the
//            step's vectors are staged in shared memory sixteen rows at a time (eight for
//            heads wider than 128);
//   finish   (row, head) in parallel: the head's output divided by its root mean square,
//            times a weight, times the sigmoid of a gate.
//
// Everything here is float whatever the activation type is: the projections arrive as float,
// and only the finished output takes the activation type.  What a thread adds and in which
// order depends on the row alone, never on where a prompt was cut or what else is in the batch.
#include "common.cuh"

#define DR_LANES 8          // threads that share one value channel
#define DR_COLS 16          // value channels a block
#define DR_MAX_D 256

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// proj: [rows, stride] float with r, k, v, gate, a at column offsets 0, HD, 2HD, 3HD, 4HD and the
// decay's inner projection (`inner` wide) at 5HD.  decay_scale is exp(-1/2) for this rule.
__global__ void delta_prepare_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ w2, const float* __restrict__ w0,
                                     const float* __restrict__ a_bias, float* __restrict__ decay, float* __restrict__ unit,
                                     float* __restrict__ removal, float* __restrict__ dots, int H, int D, int inner, float decay_scale,
                                     float key_eps) {
    extern __shared__ float th[];        // tanh of the inner projection
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, HD = H * D;
    const float* p = proj + (size_t)row * stride;
    for (int j = threadIdx.x; j < inner; j += blockDim.x) th[j] = tanhf(p[5 * HD + j]);
    __syncthreads();
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    float r = 0.0f, k = 0.0f, a = 0.0f, w = 0.0f;
    if (mine) {
        r = p[c];
        k = p[HD + c];
        a = sigmoid_f(p[4 * HD + c] + a_bias[c]);
        float z = 0.0f;
        const float* wr = w2 + (size_t)c * inner;
        for (int j = 0; j < inner; j++) z = fmaf(wr[j], th[j], z);
        w = expf(-decay_scale * sigmoid_f(z + w0[c]));
    }
    const float kk = block_sum(k * k, scratch);
    const float u = k / sqrtf(kk + key_eps);
    const float au = a * u;
    const float r_au = block_sum(r * au, scratch);
    const float r_k = block_sum(r * k, scratch);
    if (mine) {
        const size_t o = (size_t)row * HD + c;
        decay[o] = w;
        unit[o] = u;
        removal[o] = au;
    }
    if (threadIdx.x == 0) {
        dots[((size_t)row * H + head) * 2] = r_au;
        dots[((size_t)row * H + head) * 2 + 1] = r_k;
    }
}

template <int R, int DR_STEPS>   // key channels a thread (D <= 8 R) and rows staged at a time
__global__ void __launch_bounds__(DR_LANES * DR_COLS)
delta_scan_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ decay, const float* __restrict__ unit,
                  const float* __restrict__ removal, const float* __restrict__ dots, float* __restrict__ state,
                  const int* __restrict__ seq_rows, const int* __restrict__ seq_slot, float* __restrict__ out, int H, int D, int n_slots,
                  int write_state) {
    constexpr int DP = DR_LANES * R;
    __shared__ __align__(16) float sw[DR_STEPS][DP], su[DR_STEPS][DP], sb[DR_STEPS][DP], sr[DR_STEPS][DP], sk[DR_STEPS][DP];
    __shared__ float sv[DR_STEPS][DR_COLS], sd[DR_STEPS][2];
    pdl_launch_dependents();
    pdl_wait();
    const int sq = blockIdx.x, head = blockIdx.y, HD = H * D;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    if (slot < 0 || slot >= n_slots || n_new <= 0) return;
    const int lane = threadIdx.x % DR_LANES, col = threadIdx.x / DR_LANES;
    const int j = blockIdx.z * DR_COLS + col;
    const bool col_ok = j < D;
    float* S = state + ((size_t)slot * H + head) * D * D;
    float s[R];
#pragma unroll
    for (int q = 0; q < R; q++) {
        const int i = lane * R + q;
        s[q] = col_ok && i < D ? S[(size_t)i * D + j] : 0.0f;
    }
    for (int t0 = 0; t0 < n_new; t0 += DR_STEPS) {
        const int steps = min(DR_STEPS, n_new - t0);
        __syncthreads();
        for (int e = threadIdx.x; e < steps * DP; e += blockDim.x) {
            const int t = e / DP, i = e - t * DP;
            const bool in = i < D;
            const size_t row = (size_t)(row0 + t0 + t);
            const size_t o = row * HD + (size_t)head * D + i;
            sw[t][i] = in ? decay[o] : 0.0f;
            su[t][i] = in ? unit[o] : 0.0f;
            sb[t][i] = in ? removal[o] : 0.0f;
            sr[t][i] = in ? proj[row * stride + (size_t)head * D + i] : 0.0f;
            sk[t][i] = in ? proj[row * stride + HD + (size_t)head * D + i] : 0.0f;
        }
        for (int e = threadIdx.x; e < steps * DR_COLS; e += blockDim.x) {
            const int t = e / DR_COLS, cc = e - t * DR_COLS, jj = blockIdx.z * DR_COLS + cc;
            sv[t][cc] = jj < D ? proj[(size_t)(row0 + t0 + t) * stride + 2 * HD + (size_t)head * D + jj] : 0.0f;
        }
        for (int e = threadIdx.x; e < steps * 2; e += blockDim.x)
            sd[e / 2][e % 2] = dots[((size_t)(row0 + t0 + e / 2) * H + head) * 2 + e % 2];
        __syncthreads();
        for (int t = 0; t < steps; t++) {
            float rws = 0.0f, us = 0.0f;
#pragma unroll
            for (int q = 0; q < R; q++) {
                const int i = lane * R + q;
                rws = fmaf(sr[t][i] * sw[t][i], s[q], rws);
                us = fmaf(su[t][i], s[q], us);
            }
#pragma unroll
            for (int o = DR_LANES / 2; o > 0; o >>= 1) {
                rws += __shfl_xor_sync(0xffffffffu, rws, o);
                us += __shfl_xor_sync(0xffffffffu, us, o);
            }
            const float v = sv[t][col];
#pragma unroll
            for (int q = 0; q < R; q++) {
                const int i = lane * R + q;
                s[q] = fmaf(sk[t][i], v, fmaf(-sb[t][i], us, sw[t][i] * s[q]));
            }
            if (lane == 0 && col_ok)
                out[(size_t)(row0 + t0 + t) * HD + (size_t)head * D + j] = fmaf(sd[t][1], v, fmaf(-sd[t][0], us, rws));
        }
    }
    if (write_state) {
#pragma unroll
        for (int q = 0; q < R; q++) {
            const int i = lane * R + q;
            if (col_ok && i < D) S[(size_t)i * D + j] = s[q];
        }
    }
}

// out[row, c] = o[row, c] / rms(o[row, head(c)]) * weight[c] * sigmoid(gate[row, c]), in the activation type.
template <class T>
__global__ void delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride, const float* __restrict__ weight,
                                    T* __restrict__ out, int H, int D, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, HD = H * D;
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    const float v = mine ? o[(size_t)row * HD + c] : 0.0f;
    const float ss = block_sum(v * v, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)D + eps);
    if (mine) out[(size_t)row * HD + c] = from_f32<T>(v * scale * weight[c] * sigmoid_f(gate[(size_t)row * gate_stride + c]));
}

// A step of one row a sequence: prepare, one step of the scan and finish in one launch, a block a (row, head)
// with eight threads a value channel.  Every sum is taken by the same threads in the same order as in the three
// kernels above (thread d holds channel d in the sums over a head), so a row decoded alone and the same row in a
// prompt give the same bits.  Heads of up to 128 channels.
template <int R, class T>
__global__ void __launch_bounds__(64 * R)
delta_step_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ w2, const float* __restrict__ w0,
                  const float* __restrict__ a_bias, const float* __restrict__ norm_w, float* __restrict__ state,
                  const int* __restrict__ row_slot, T* __restrict__ out, int H, int D, int inner, float decay_scale, float key_eps,
                  float norm_eps, int n_slots, int write_state) {
    constexpr int DP = DR_LANES * R;
    extern __shared__ float sm[];
    __shared__ float scratch[32];
    float* th = sm;
    float* sw = th + ((inner + 3) & ~3);
    float *su = sw + DP, *sb = su + DP, *sr = sb + DP, *sk = sr + DP, *so = sk + DP;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, HD = H * D;
    const int slot = row_slot[row];
    if (slot < 0 || slot >= n_slots) return;
    const float* p = proj + (size_t)row * stride;
    for (int j = threadIdx.x; j < inner; j += blockDim.x) th[j] = tanhf(p[5 * HD + j]);
    __syncthreads();
    const int d = threadIdx.x, c = head * D + d;
    const bool mine = d < D;
    float r = 0.0f, k = 0.0f, a = 0.0f, w = 0.0f;
    if (mine) {
        r = p[c];
        k = p[HD + c];
        a = sigmoid_f(p[4 * HD + c] + a_bias[c]);
        float z = 0.0f;
        const float* wr = w2 + (size_t)c * inner;
        for (int j = 0; j < inner; j++) z = fmaf(wr[j], th[j], z);
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
    float* S = state + ((size_t)slot * H + head) * D * D;
    float s[R];
#pragma unroll
    for (int q = 0; q < R; q++) {
        const int i = lane * R + q;
        s[q] = col_ok && i < D ? S[(size_t)i * D + j] : 0.0f;
    }
    float rws = 0.0f, us = 0.0f;
#pragma unroll
    for (int q = 0; q < R; q++) {
        const int i = lane * R + q;
        rws = fmaf(sr[i] * sw[i], s[q], rws);
        us = fmaf(su[i], s[q], us);
    }
#pragma unroll
    for (int o = DR_LANES / 2; o > 0; o >>= 1) {
        rws += __shfl_xor_sync(0xffffffffu, rws, o);
        us += __shfl_xor_sync(0xffffffffu, us, o);
    }
    const float v = col_ok ? p[2 * HD + (size_t)head * D + j] : 0.0f;
    if (write_state) {
#pragma unroll
        for (int q = 0; q < R; q++) {
            const int i = lane * R + q;
            if (col_ok && i < D) S[(size_t)i * D + j] = fmaf(sk[i], v, fmaf(-sb[i], us, sw[i] * s[q]));
        }
    }
    if (lane == 0 && col_ok) so[j] = fmaf(r_k, v, fmaf(-r_au, us, rws));
    __syncthreads();
    const float o = mine ? so[d] : 0.0f;
    const float ss = block_sum(o * o, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)D + norm_eps);
    if (mine) out[(size_t)row * HD + c] = from_f32<T>(o * scale * norm_w[c] * sigmoid_f(p[3 * HD + c]));
}

template <class T>
static int step(const float* proj, int stride, const float* w2, const float* w0, const float* a_bias, const float* norm_w, float* state,
                const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale, float key_eps, float norm_eps, int n_slots,
                int write_state, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 128 && inner > 0 && inner <= 8192,
                 "delta_step: bad sizes rows=%d H=%d D=%d inner=%d (a head of at most 128)", rows, H, D, inner);
    BC_CHECK_ARG(stride >= 5 * H * D + inner, "delta_step: a row of %d values cannot hold five projections of %d and %d more", stride, H * D, inner);
    if (rows == 0) return BC_OK;
    const int threads = DR_LANES * ((D + 3) / 4 * 4);
    const dim3 grid(rows, H);
#define DS_CASE(R)                                                                                                                         \
    bc_launch(delta_step_kernel<R, T>, grid, dim3(threads), (size_t)(((inner + 3) & ~3) + 5 * DR_LANES * R + D) * sizeof(float), s, proj, \
              stride, w2, w0, a_bias, norm_w, state, row_slot, (T*)out, H, D, inner, decay_scale, key_eps, norm_eps, n_slots, write_state)
    if (D <= 16) DS_CASE(2);
    else if (D <= 32) DS_CASE(4);
    else if (D <= 64) DS_CASE(8);
    else DS_CASE(16);
#undef DS_CASE
    BC_LAUNCH_STATUS();
}
// One row a sequence (row r lives in slot row_slot[r]; negative: skipped, its row of `out` is left untouched):
// proj as for bc_delta_prepare, state as for bc_delta_scan, out [rows, H D] as from bc_delta_finish.
extern "C" int bc_delta_step_f32(const float* proj, int stride, const float* w2, const float* w0, const float* a_bias, const float* norm_w,
                                 float* state, const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale,
                                 float key_eps, float norm_eps, int n_slots, int write_state, cudaStream_t s) {
    return step<float>(proj, stride, w2, w0, a_bias, norm_w, state, row_slot, out, rows, H, D, inner, decay_scale, key_eps, norm_eps, n_slots,
                       write_state, s);
}
extern "C" int bc_delta_step_bf16(const float* proj, int stride, const float* w2, const float* w0, const float* a_bias, const float* norm_w,
                                  float* state, const int* row_slot, void* out, int rows, int H, int D, int inner, float decay_scale,
                                  float key_eps, float norm_eps, int n_slots, int write_state, cudaStream_t s) {
    return step<bf16>(proj, stride, w2, w0, a_bias, norm_w, state, row_slot, out, rows, H, D, inner, decay_scale, key_eps, norm_eps, n_slots,
                      write_state, s);
}

static int threads_for(int D) { return ((D + 31) / 32) * 32; }

extern "C" int bc_delta_prepare(const float* proj, int stride, const float* w2, const float* w0, const float* a_bias, float* decay, float* unit,
                                float* removal, float* dots, int rows, int H, int D, int inner, float decay_scale, float key_eps,
                                cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 1024 && inner > 0 && inner <= 8192,
                 "delta_prepare: bad sizes rows=%d H=%d D=%d inner=%d", rows, H, D, inner);
    BC_CHECK_ARG(stride >= 5 * H * D + inner, "delta_prepare: a row of %d values cannot hold five projections of %d and %d more", stride, H * D, inner);
    if (rows == 0) return BC_OK;
    bc_launch(delta_prepare_kernel, dim3(rows, H), dim3(threads_for(D)), (size_t)inner * sizeof(float), s, proj, stride, w2, w0, a_bias, decay,
              unit, removal, dots, H, D, inner, decay_scale, key_eps);
    BC_LAUNCH_STATUS();
}

// state: [n_slots, H, D, D] float.  Sequence s owns rows seq_rows[s] .. seq_rows[s + 1] and lives in
// slot seq_slot[s] (negative: skipped, its rows of `out` are left untouched).  write_state 0 leaves
// the state as it was.
extern "C" int bc_delta_scan(const float* proj, int stride, const float* decay, const float* unit, const float* removal, const float* dots,
                             float* state, const int* seq_rows, const int* seq_slot, float* out, int seqs, int H, int D, int n_slots,
                             int write_state, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 2147483647 && H > 0 && H <= 65535 && D > 0 && D <= DR_MAX_D,
                 "delta_scan: bad sizes seqs=%d H=%d D=%d (a head of at most %d)", seqs, H, D, DR_MAX_D);
    if (seqs == 0) return BC_OK;
    const dim3 grid(seqs, H, (D + DR_COLS - 1) / DR_COLS), block(DR_LANES * DR_COLS);
#define DR_CASE(R, STEPS)                                                                                                                      \
    bc_launch(delta_scan_kernel<R, STEPS>, grid, block, 0, s, proj, stride, decay, unit, removal, dots, state, seq_rows, seq_slot, out, H, D, \
              n_slots, write_state)
    if (D <= 16) DR_CASE(2, 16);
    else if (D <= 32) DR_CASE(4, 16);
    else if (D <= 64) DR_CASE(8, 16);
    else if (D <= 128) DR_CASE(16, 16);
    else DR_CASE(32, 8);
#undef DR_CASE
    BC_LAUNCH_STATUS();
}

template <class T>
static int finish(const float* o, const float* gate, int gate_stride, const float* weight, void* out, int rows, int H, int D, float eps,
                  cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && H > 0 && H <= 65535 && D > 0 && D <= 1024, "delta_finish: bad sizes rows=%d H=%d D=%d", rows, H, D);
    if (rows == 0) return BC_OK;
    bc_launch(delta_finish_kernel<T>, dim3(rows, H), dim3(threads_for(D)), 0, s, o, gate, gate_stride, weight, (T*)out, H, D, eps);
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
