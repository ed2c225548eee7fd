// Recurrent mixers whose state decays channel by channel and takes an outer product a token:
//
//     S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T        o_t = f S_t^T q_t + d v_t
//
// per head, with S [N, P] (N key channels, P value channels) in float, carried from token to token for every
// sequence.  Two designs are this recurrence:
//   - gated linear attention: a_t a vector of N decays, c = 1, d = 0, f = N^(-1/2), q, k, v per head;
//   - the state-space dual form (Mamba-2): a_t = exp(-exp(A_log) dt_t) one number a head, c_t = dt_t, k = B and
//     q = C shared by the heads of a group, v = x, d = D of the head.
// Everything here is float: decays, step sizes, the state and all sums.
//
// Kernels:
//   scan           the recurrence over every sequence's rows in time order
//   ssd_prepare    causal convolution with bias and silu over [x | B | C], its last inputs kept per sequence;
//                  dt = softplus(. + dt_bias) and the decay exp(-exp(A_log) dt)
//   gla_decay      sigmoid(z)^(1/tau), z = W_2 inner + b, as exp(-softplus(-z) / tau)
//   gated_norm     a row in equal parts, each over its root mean square, times a weight, the gate silu(g) before
//                  or after the norm, a factor on the result; float in, activation type out
#include "common.cuh"

#define SCAN_NT 8          // threads that share a value channel, each with every eighth key channel
#define SCAN_MAX_N 256
#define SCAN_PT 32         // value channels a block: two a thread

__device__ __forceinline__ void scan_copy4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_copy16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void scan_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT> __device__ __forceinline__ void scan_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory"); }

// A block takes (a slice of 32 value channels, head, sequence): thread (tn, pl) keeps S[n][p] for n = tn, tn + 8, ... and
// p = p0 + pl, p0 + 16 + pl in registers over the sequence's rows.  The state lies in memory value channel by value
// channel, [slot][head][P][N], so that the eight threads of a channel read neighbouring values.  Rows are staged R at a time
// in shared memory by asynchronous copies, the next R on their way while these are worked on (16 bytes a copy where every
// run starts on such a border: VEC).  A staged row of q, k or decays is NP = 8 NJ values long, zeros past the N that exist,
// so that the loop over a thread's key channels has no test in it: with one, every channel's loads waited behind the
// branch of the channel before (75 clocks a channel measured, 1,500 a step of 128 channels).  The sums of a step depend on
// the sizes alone: the same bits whether a row comes in a prompt or alone.
template <int NJ, bool VECTOR_DECAY, bool VEC>
__global__ void __launch_bounds__(128)
linear_scan_kernel(const float* __restrict__ q, int q_stride, int q_rep, const float* __restrict__ k, int k_stride, int k_rep,
                   const float* __restrict__ v, int v_stride, const float* __restrict__ decay, int d_stride,
                   const float* __restrict__ kscale, int c_stride, const float* __restrict__ skip, float out_scale,
                   float* __restrict__ state, const int* __restrict__ seq_rows, const int* __restrict__ seq_slot, float* __restrict__ out,
                   int H, int N, int P, int R, int n_slots, int write_state) {
    extern __shared__ __align__(16) float staged[];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(q); PDL_FRESH(k); PDL_FRESH(v); PDL_FRESH(decay); PDL_FRESH(kscale);
    const int sidx = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * SCAN_PT;
    const int slot = seq_slot[sidx];
    const int row0 = seq_rows[sidx], n_rows = seq_rows[sidx + 1] - row0;
    if (slot < 0 || slot >= n_slots || n_rows <= 0) return;
    const int tn = threadIdx.x % SCAN_NT, pl = threadIdx.x / SCAN_NT;         // 8 x 16 threads
    const int pa = p0 + pl, pb = p0 + 16 + pl;
    const bool live_a = pa < P, live_b = pb < P;
    float* sa = state + (((size_t)slot * H + h) * P + (live_a ? pa : 0)) * N;
    float* sb = state + (((size_t)slot * H + h) * P + (live_b ? pb : 0)) * N;
    float Sa[NJ], Sb[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int n = tn + SCAN_NT * j;
        Sa[j] = live_a && n < N ? sa[n] : 0.0f;
        Sb[j] = live_b && n < N ? sb[n] : 0.0f;
    }
    const float dskip = skip ? skip[h] : 0.0f;
    // A stage: R rows of q, of k, of the decays (VECTOR_DECAY), of the block's 32 values, and the rows' two scalars.
    constexpr int NP = SCAN_NT * NJ;
    const int n_arrays = VECTOR_DECAY ? 3 : 2;
    const int stage_floats = R * (n_arrays * NP + SCAN_PT + 2);
    if (NP != N) {
        // The padding of every staged row, once: no copy ever lands there.
        const int pad = NP - N;
        for (int i = threadIdx.x; i < 2 * n_arrays * R * pad; i += 128) {
            const int row = i / pad, c = N + i - row * pad;           // row counts over stages, arrays and rows
            const int stage = row / (n_arrays * R), in_stage = row - stage * (n_arrays * R);
            staged[(size_t)stage * stage_floats + (size_t)in_stage * NP + c] = 0.0f;
        }
    }
    const float* qh = q + (size_t)(h / q_rep) * N;
    const float* kh = k + (size_t)(h / k_rep) * N;
    const float* dh = decay + (VECTOR_DECAY ? (size_t)h * N : (size_t)h);
    const float* vh = v + (size_t)h * P + p0;
    const int pv = min(SCAN_PT, P - p0);                    // values of this block a row
    auto issue = [&](int chunk, int stage) {
        const int t0 = chunk * R, nt = min(R, n_rows - t0);
        float* sq = staged + (size_t)stage * stage_floats;
        float* sk = sq + R * NP;
        float* sd = sk + R * NP;
        float* sv = sq + n_arrays * R * NP;
        float* sc = sv + R * SCAN_PT;
        const size_t r0 = (size_t)(row0 + t0);
        if (VEC) {
            const int n4 = N / 4, pv4 = pv / 4;
            for (int i = threadIdx.x; i < nt * n4; i += 128) {
                const int t = i / n4, c = 4 * (i - t * n4);
                scan_copy16(sq + t * NP + c, qh + (r0 + t) * q_stride + c);
                scan_copy16(sk + t * NP + c, kh + (r0 + t) * k_stride + c);
                if (VECTOR_DECAY) scan_copy16(sd + t * NP + c, dh + (r0 + t) * d_stride + c);
            }
            for (int i = threadIdx.x; i < nt * pv4; i += 128) {
                const int t = i / pv4, c = 4 * (i - t * pv4);
                scan_copy16(sv + t * SCAN_PT + c, vh + (r0 + t) * v_stride + c);
            }
        } else {
            for (int i = threadIdx.x; i < nt * N; i += 128) {
                const int t = i / N, c = i - t * N;
                scan_copy4(sq + t * NP + c, qh + (r0 + t) * q_stride + c);
                scan_copy4(sk + t * NP + c, kh + (r0 + t) * k_stride + c);
                if (VECTOR_DECAY) scan_copy4(sd + t * NP + c, dh + (r0 + t) * d_stride + c);
            }
            for (int i = threadIdx.x; i < nt * pv; i += 128) {
                const int t = i / pv, c = i - t * pv;
                scan_copy4(sv + t * SCAN_PT + c, vh + (r0 + t) * v_stride + c);
            }
        }
        if ((int)threadIdx.x < nt) {
            if (kscale) scan_copy4(sc + threadIdx.x, kscale + (r0 + threadIdx.x) * c_stride + h);
            else sc[threadIdx.x] = 1.0f;
            if (!VECTOR_DECAY) scan_copy4(sc + R + threadIdx.x, dh + (r0 + threadIdx.x) * d_stride);
        }
    };
    const int chunks = (n_rows + R - 1) / R;
    issue(0, 0);
    scan_commit();
    for (int chunk = 0; chunk < chunks; chunk++) {
        if (chunk + 1 < chunks) issue(chunk + 1, (chunk + 1) & 1);
        scan_commit();
        scan_wait<1>();
        __syncthreads();
        const int t0 = chunk * R, nt = min(R, n_rows - t0);
        const float* sq = staged + (size_t)(chunk & 1) * stage_floats + tn;
        const float* sk = sq + R * NP;
        const float* sd = sk + R * NP;
        const float* sv = staged + (size_t)(chunk & 1) * stage_floats + n_arrays * R * NP;
        const float* sc = sv + R * SCAN_PT;
        // Two steps are unrolled together, so that one's shuffles and store pass while the other's loads and sums run.
#pragma unroll 2
        for (int t = 0; t < nt; t++) {
            const float va = pl < pv ? sv[t * SCAN_PT + pl] : 0.0f, vb = 16 + pl < pv ? sv[t * SCAN_PT + 16 + pl] : 0.0f;
            const float ca = sc[t] * va, cb = sc[t] * vb;
            const float a0 = VECTOR_DECAY ? 0.0f : sc[R + t];
            float oa = 0.0f, ob = 0.0f, oa2 = 0.0f, ob2 = 0.0f;      // even and odd channels apart: two chains half as long
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const float a = VECTOR_DECAY ? sd[t * NP + SCAN_NT * j] : a0, kk = sk[t * NP + SCAN_NT * j], qq = sq[t * NP + SCAN_NT * j];
                Sa[j] = fmaf(a, Sa[j], kk * ca);
                Sb[j] = fmaf(a, Sb[j], kk * cb);
                if (j & 1) {
                    oa2 = fmaf(Sa[j], qq, oa2);
                    ob2 = fmaf(Sb[j], qq, ob2);
                } else {
                    oa = fmaf(Sa[j], qq, oa);
                    ob = fmaf(Sb[j], qq, ob);
                }
            }
            oa += oa2;
            ob += ob2;
            oa += __shfl_xor_sync(0xffffffffu, oa, 1);
            ob += __shfl_xor_sync(0xffffffffu, ob, 1);
            oa += __shfl_xor_sync(0xffffffffu, oa, 2);
            ob += __shfl_xor_sync(0xffffffffu, ob, 2);
            oa += __shfl_xor_sync(0xffffffffu, oa, 4);
            ob += __shfl_xor_sync(0xffffffffu, ob, 4);
            float* o = out + (size_t)(row0 + t0 + t) * H * P + (size_t)h * P;
            if (live_a && tn == 0) o[pa] = fmaf(dskip, va, out_scale * oa);
            if (live_b && tn == 1) o[pb] = fmaf(dskip, vb, out_scale * ob);
        }
        __syncthreads();          // all have read the stage before the copies of the chunk after next land in it
    }
    if (write_state) {
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int n = tn + SCAN_NT * j;
            if (live_a && n < N) sa[n] = Sa[j];
            if (live_b && n < N) sb[n] = Sb[j];
        }
    }
}

template <int NJ, bool VD, bool VEC>
static cudaError_t scan_launch_one(dim3 grid, size_t smem, cudaStream_t s, const float* q, int q_stride, int q_rep, const float* k, int k_stride,
                                   int k_rep, const float* v, int v_stride, const float* decay, int d_stride, const float* kscale, int c_stride,
                                   const float* skip, float out_scale, float* state, const int* seq_rows, const int* seq_slot, float* out, int H,
                                   int N, int P, int R, int n_slots, int write_state) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel<NJ, VD, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    return bc_launch(linear_scan_kernel<NJ, VD, VEC>, grid, dim3(128), smem, s, q, q_stride, q_rep, k, k_stride, k_rep, v, v_stride, decay, d_stride,
                     kscale, c_stride, skip, out_scale, state, seq_rows, seq_slot, out, H, N, P, R, n_slots, write_state);
}

template <bool VD, bool VEC>
static int scan_launch(int NJ, dim3 grid, size_t smem, cudaStream_t s, const float* q, int q_stride, int q_rep, const float* k, int k_stride,
                       int k_rep, const float* v, int v_stride, const float* decay, int d_stride, const float* kscale, int c_stride,
                       const float* skip, float out_scale, float* state, const int* seq_rows, const int* seq_slot, float* out, int H, int N,
                       int P, int R, int n_slots, int write_state) {
    cudaError_t e = cudaSuccess;
#define SCAN_CASE(J)                                                                                                                         \
    case J:                                                                                                                                  \
        e = scan_launch_one<J, VD, VEC>(grid, smem, s, q, q_stride, q_rep, k, k_stride, k_rep, v, v_stride, decay, d_stride, kscale, c_stride, \
                                        skip, out_scale, state, seq_rows, seq_slot, out, H, N, P, R, n_slots, write_state);                  \
        break;
    switch (NJ) {
        SCAN_CASE(1) SCAN_CASE(2) SCAN_CASE(4) SCAN_CASE(8) SCAN_CASE(12) SCAN_CASE(16) SCAN_CASE(24) SCAN_CASE(32)
    }
#undef SCAN_CASE
    if (e != cudaSuccess) {
        bc_set_error("linear_scan: %s", cudaGetErrorString(e));
        return (int)e;
    }
    BC_LAUNCH_STATUS();
}

// q, k: row r's vector for head h at base + r * stride + (h / rep) * N (rep heads share one); v: at v + r * v_stride + h * P;
// decay: N values a head at decay + r * d_stride + h * N (vector_decay) or one at decay + r * d_stride + h; kscale (may be null):
// one factor a head on the key at kscale + r * c_stride + h; skip (may be null): [H].  state: [slots, H, P, N]; out: [rows, H P].
// Sequence i owns rows seq_rows[i] .. seq_rows[i + 1] and lives in slot seq_slot[i] (negative: skipped, its rows of out untouched).
extern "C" int bc_linear_scan(const float* q, int q_stride, int q_rep, const float* k, int k_stride, int k_rep, const float* v, int v_stride,
                              const float* decay, int d_stride, int vector_decay, const float* kscale, int c_stride, const float* skip,
                              float out_scale, float* state, const int* seq_rows, const int* seq_slot, float* out, int seqs, int H, int N, int P,
                              int n_slots, int write_state, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && H > 0 && H <= 65535 && P > 0, "linear_scan: bad sizes seqs=%d H=%d P=%d", seqs, H, P);
    BC_CHECK_ARG(N > 0 && N <= SCAN_MAX_N, "linear_scan: %d key channels are outside 1 to %d", N, SCAN_MAX_N);
    BC_CHECK_ARG(q_rep > 0 && k_rep > 0, "linear_scan: bad sharing of q (%d) or k (%d)", q_rep, k_rep);
    if (seqs == 0) return BC_OK;
    int nj = (N + SCAN_NT - 1) / SCAN_NT;
    const int have[] = {1, 2, 4, 8, 12, 16, 24, 32};
    for (int c : have)
        if (c >= nj) { nj = c; break; }
    // Rows a stage: sixteen, eight for the widest heads (two stages of q, k and decays must fit beside other blocks).
    const int R = N > 128 ? 8 : 16;
    const size_t smem = 2 * (size_t)R * ((vector_decay ? 3 : 2) * SCAN_NT * nj + SCAN_PT + 2) * sizeof(float);
    // 16 bytes a copy where every run of every row starts on a 16-byte border and is a multiple of 16 bytes long.
    const bool vec = N % 4 == 0 && P % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 && (!vector_decay || d_stride % 4 == 0) &&
                     (uintptr_t)q % 16 == 0 && (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0 && (!vector_decay || (uintptr_t)decay % 16 == 0);
    dim3 grid((P + SCAN_PT - 1) / SCAN_PT, H, seqs);
#define SCAN_GO(VD, VEC)                                                                                                                    \
    return scan_launch<VD, VEC>(nj, grid, smem, s, q, q_stride, q_rep, k, k_stride, k_rep, v, v_stride, decay, d_stride, kscale, c_stride, skip, \
                                out_scale, state, seq_rows, seq_slot, out, H, N, P, R, n_slots, write_state)
    if (vector_decay) {
        if (vec) SCAN_GO(true, true);
        SCAN_GO(true, false);
    }
    if (vec) SCAN_GO(false, true);
    SCAN_GO(false, false);
#undef SCAN_GO
}

// ------------------------------------------------------------------------------- ssd_prepare
// proj: [rows, stride] float with the convolution's C channels at column `conv_at` and H step sizes at column `dt_at`.
// Thread c < C walks a tile of a sequence's rows with the last taps - 1 inputs in registers: out[r][c] =
// silu(bias[c] + sum_j w[j][c] in[t - taps + 1 + j]); inputs before the step's first row come from `tail`
// [slots, taps - 1, C], zeros at a sequence's start since the cache clears a slot's state.  The block of a
// sequence's first tile is the only reader of the old tail and writes the new one when it is done.  Threads
// C .. C + H - 1 take the step sizes: dtda[r] = (dt[0..H), decay[0..H)).
#define SSD_TILE 32
#define SSD_MAX_TAPS 9
__global__ void __launch_bounds__(128)
ssd_prepare_kernel(const float* __restrict__ proj, int stride, int conv_at, int dt_at, const float* __restrict__ weight_t,
                   const float* __restrict__ bias, const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ tail,
                   const int* __restrict__ seq_rows, const int* __restrict__ seq_slot, float* __restrict__ xbc, float* __restrict__ dtda, int C,
                   int H, int taps, int n_slots, int write_tail) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int sidx = blockIdx.z, tile = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = seq_slot[sidx];
    const int row0 = seq_rows[sidx], n_rows = seq_rows[sidx + 1] - row0;
    const int t_begin = tile * SSD_TILE;
    if (slot < 0 || slot >= n_slots || t_begin >= n_rows || c >= C + H) return;
    const int t_end = min(n_rows, t_begin + SSD_TILE);
    if (c >= C) {
        const int h = c - C;
        const float b = dt_bias[h], a = -expf(a_log[h]);
        for (int t = t_begin; t < t_end; t++) {
            const float z = proj[(size_t)(row0 + t) * stride + dt_at + h] + b;
            const float dt = z > 20.0f ? z : log1pf(expf(z));
            float* o = dtda + (size_t)(row0 + t) * 2 * H;
            o[h] = dt;
            o[H + h] = expf(a * dt);
        }
        return;
    }
    const int past = taps - 1;
    float w[SSD_MAX_TAPS], hist[SSD_MAX_TAPS - 1], old[SSD_MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < SSD_MAX_TAPS; j++) w[j] = j < taps ? weight_t[(size_t)j * C + c] : 0.0f;
    float* tl = tail + (size_t)slot * past * C + c;
    // hist[i] is the input of relative time t_begin - past + i.
#pragma unroll
    for (int i = 0; i < SSD_MAX_TAPS - 1; i++) {
        hist[i] = 0.0f;
        old[i] = 0.0f;
        if (i < past) {
            const int t = t_begin - past + i;
            if (t >= 0) hist[i] = proj[(size_t)(row0 + t) * stride + conv_at + c];
            else if (tile == 0) hist[i] = old[i] = tl[(size_t)i * C];      // t_begin is 0 here: the old tail as it is
        }
    }
    const float b = bias ? bias[c] : 0.0f;
    for (int t = t_begin; t < t_end; t++) {
        const float x = proj[(size_t)(row0 + t) * stride + conv_at + c];
        float acc = b;
#pragma unroll
        for (int j = 0; j < SSD_MAX_TAPS - 1; j++)
            if (j < past) acc = fmaf(w[j], hist[j], acc);
        acc = fmaf(w[past], x, acc);
#pragma unroll
        for (int j = 0; j < SSD_MAX_TAPS - 2; j++)
            if (j + 1 < past) hist[j] = hist[j + 1];
        if (past > 0) hist[past - 1] = x;
        xbc[(size_t)(row0 + t) * C + c] = acc / (1.0f + expf(-acc));
    }
    if (tile == 0 && write_tail) {
        // The new tail: the last `past` inputs of the sequence, of which the step may have brought fewer.
#pragma unroll
        for (int i = 0; i < SSD_MAX_TAPS - 1; i++) {
            if (i < past) {
                const int t = n_rows - past + i;
                tl[(size_t)i * C] = t >= 0 ? proj[(size_t)(row0 + t) * stride + conv_at + c] : old[i + n_rows];
            }
        }
    }
}

// weight_t: [taps, C] (tap by tap; the last is the current token's); bias: [C] or null; dt_bias, a_log: [H];
// tail: [slots, taps - 1, C]; xbc: [rows, C]; dtda: [rows, 2 H].
extern "C" int bc_ssd_prepare(const float* proj, int stride, int conv_at, int dt_at, const float* weight_t, const float* bias, const float* dt_bias,
                              const float* a_log, float* tail, const int* seq_rows, const int* seq_slot, float* xbc, float* dtda, int seqs,
                              int max_new, int C, int H, int taps, int n_slots, int write_tail, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && max_new >= 0 && C > 0 && H > 0, "ssd_prepare: bad sizes seqs=%d max_new=%d C=%d H=%d", seqs, max_new, C, H);
    BC_CHECK_ARG(taps >= 1 && taps <= SSD_MAX_TAPS, "ssd_prepare: %d taps are outside 1 to %d", taps, SSD_MAX_TAPS);
    if (seqs == 0 || max_new == 0) return BC_OK;
    const int tiles = (max_new + SSD_TILE - 1) / SSD_TILE;
    BC_CHECK_ARG(tiles <= 65535, "ssd_prepare: %d rows a sequence are too many", max_new);
    dim3 grid((C + H + 127) / 128, tiles, seqs);
    bc_launch(ssd_prepare_kernel, grid, dim3(128), 0, s, proj, stride, conv_at, dt_at, weight_t, bias, dt_bias, a_log, tail, seq_rows, seq_slot, xbc,
              dtda, C, H, taps, n_slots, write_tail);
    BC_LAUNCH_STATUS();
}

// --------------------------------------------------------------------------------- gla_decay
// decay[r][c] = sigmoid(z)^(1/tau) with z = sum_i w2t[i][c] inner[r][i] + b[c], computed as exp(-softplus(-z) / tau)
// so that no logarithm of a rounded sigmoid is taken.  One block a row; the inner vector is staged in shared memory.
__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ proj, int stride, int inner_at, const float* __restrict__ w2t, const float* __restrict__ b,
                 float* __restrict__ decay, int W, int rank, float inv_tau) {
    extern __shared__ float inner[];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(proj);
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) inner[i] = proj[(size_t)r * stride + inner_at + i];
    __syncthreads();
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float z = b[c];
#pragma unroll 8
        for (int i = 0; i < rank; i++) z = fmaf(w2t[(size_t)i * W + c], inner[i], z);      // eight loads asked for together; the sum's order stays
        const float m = -z;                                          // softplus(m) = max(m, 0) + log1p(exp(-|m|))
        const float sp = fmaxf(m, 0.0f) + log1pf(expf(-fabsf(m)));
        decay[(size_t)r * W + c] = expf(-sp * inv_tau);
    }
}

// proj: [rows, stride] float with the inner projection's `rank` values at column inner_at; w2t: [rank, W]; b: [W]; decay: [rows, W].
extern "C" int bc_gla_decay(const float* proj, int stride, int inner_at, const float* w2t, const float* b, float* decay, int rows, int W, int rank,
                            float tau, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && W > 0 && rank > 0 && rank <= 8192 && tau > 0.0f, "gla_decay: bad sizes rows=%d W=%d rank=%d tau=%g", rows, W, rank, (double)tau);
    if (rows == 0) return BC_OK;
    bc_launch(gla_decay_kernel, dim3(rows), dim3(W >= 1024 ? 256 : 128), (size_t)rank * sizeof(float), s, proj, stride, inner_at, w2t, b, decay, W,
              rank, 1.0f / tau);
    BC_LAUNCH_STATUS();
}

// -------------------------------------------------------------------------------- gated_norm
// y: [rows, W] float; gate: row r's at gate + r * g_stride; weight: `period` values, repeated over the row (period = W: one
// a column; period = W / parts: shared by the parts); row_slot (may be null): rows whose slot is negative give zeros.  Block (part, row): z = y (* silu(g) if gate_first); z over the root mean
// square of the part, eps inside the root; times weight (times silu(g) if not gate_first); times factor.
template <class T>
__global__ void __launch_bounds__(256)
gated_norm_kernel(const float* __restrict__ y, const float* __restrict__ gate, int g_stride, const float* __restrict__ weight, int period,
                  const int* __restrict__ row_slot, T* __restrict__ out, int W, int part, float eps, int gate_first, float factor) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(y); PDL_FRESH(gate);
    const int r = blockIdx.y, c0 = blockIdx.x * part;
    if (row_slot != nullptr && row_slot[r] < 0) {
        // A row of no sequence: nothing wrote its y (the recurrence walks sequences), so it is not read; zeros go on.
        for (int c = threadIdx.x; c < part; c += blockDim.x) out[(size_t)r * W + c0 + c] = from_f32<T>(0.0f);
        return;
    }
    const float* yr = y + (size_t)r * W + c0;
    const float* gr = gate + (size_t)r * g_stride + c0;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < part; c += blockDim.x) {
        float z = yr[c];
        if (gate_first) {
            const float g = gr[c];
            z *= g / (1.0f + expf(-g));
        }
        ss = fmaf(z, z, ss);
    }
    const float scale = factor / sqrtf(block_sum(ss, scratch) / (float)part + eps);
    for (int c = threadIdx.x; c < part; c += blockDim.x) {
        const float g = gr[c];
        const float sg = g / (1.0f + expf(-g));
        const float z = gate_first ? yr[c] * sg : yr[c];
        const float o = z * scale * weight[(c0 + c) % period];
        out[(size_t)r * W + c0 + c] = from_f32<T>(gate_first ? o : o * sg);
    }
}

template <class T>
static int gated_norm(const float* y, const float* gate, int g_stride, const float* weight, int period, const int* row_slot, void* out, int rows,
                      int W, int parts, float eps, int gate_first, float factor, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && rows <= 2147483647 && W > 0 && parts > 0 && parts <= 65535 && W % parts == 0, "gated_norm: bad sizes rows=%d W=%d parts=%d", rows, W, parts);
    BC_CHECK_ARG(period > 0 && (period == W || period == W / parts), "gated_norm: a weight of %d values fits neither the row nor a part", period);
    if (rows == 0) return BC_OK;
    const int part = W / parts;
    const int threads = part >= 1024 ? 256 : part >= 256 ? 128 : part >= 64 ? 64 : 32;       // by the part's width alone
    // More rows than a grid's second dimension holds go in turns.
    for (int at = 0; at < rows; at += 65535) {
        const int n = rows - at < 65535 ? rows - at : 65535;
        bc_launch(gated_norm_kernel<T>, dim3(parts, n), dim3(threads), 0, s, y + (size_t)at * W, gate + (size_t)at * g_stride, g_stride, weight, period,
                  row_slot ? row_slot + at : nullptr, (T*)out + (size_t)at * W, W, part, eps, gate_first, factor);
    }
    BC_LAUNCH_STATUS();
}
extern "C" int bc_gated_norm_f32(const float* y, const float* gate, int g_stride, const float* weight, int period, const int* row_slot, void* out,
                                 int rows, int W, int parts, float eps, int gate_first, float factor, cudaStream_t s) {
    return gated_norm<float>(y, gate, g_stride, weight, period, row_slot, out, rows, W, parts, eps, gate_first, factor, s);
}
extern "C" int bc_gated_norm_bf16(const float* y, const float* gate, int g_stride, const float* weight, int period, const int* row_slot, void* out,
                                  int rows, int W, int parts, float eps, int gate_first, float factor, cudaStream_t s) {
    return gated_norm<bf16>(y, gate, g_stride, weight, period, row_slot, out, rows, W, parts, eps, gate_first, factor, s);
}
