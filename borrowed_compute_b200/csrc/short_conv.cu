// A short causal convolution over time on every channel, added to its own input:
//   out[t, c] = h[t, c] + sum_{j < taps} w[j, c] * h[t - (taps - 1 - j), c]
// with zeros before a sequence's first position.  The last taps - 1 inputs of a sequence
// are state that outlives the step: tail[slot][i][c] holds the input at position
// start - (taps - 1) + i, where `start` is how many positions the slot held before this
// step (a slot handed out anew holds zeros there, which is the convolution's padding).
//
// Every (row, channel) is one thread's sum of `taps` terms in ascending j, so a row's result
// is the same bits whether it came in a prompt, in a portion of one, or alone.  The products
// and the sum are float; inputs, outputs and the tail have the activation type.
//
// Two launches a prompt step: the convolution (which only reads the tail) and then the new
// tail.  A step of one row a sequence does both in one launch: a channel of a sequence is
// then one thread's alone.
#include "common.cuh"

#define SC_THREADS 256

// V values of the activation type, as floats and back: one 16-byte access where V * sizeof(T) is 16.
template <class T, int V> __device__ __forceinline__ void load_values(const T* p, float* v) {
    if constexpr (V == 1) {
        v[0] = to_f32(p[0]);
    } else if constexpr (sizeof(T) == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}
template <class T, int V> __device__ __forceinline__ void store_values(T* p, const float* v) {
    if constexpr (V == 1) {
        p[0] = from_f32<T>(v[0]);
    } else if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        static_assert(sizeof(T) == 4 || V == 1 || V == 4 || V == 8, "bf16 values go four or eight at a time");
        uint32_t w[V / 2];
#pragma unroll
        for (int i = 0; i < V / 2; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        if constexpr (V == 8) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
        else *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
    }
}

// A thread takes V neighbouring channels of one row (V = 16 bytes' worth where the width allows, else 1).
template <class T, int V>
__global__ void __launch_bounds__(SC_THREADS)
short_conv_kernel(const T* __restrict__ h, const float* __restrict__ w, T* __restrict__ tail, const int* __restrict__ seq_rows,
                  const int* __restrict__ seq_slot, T* __restrict__ out, int E, int taps, int n_slots, int update_tail) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(h);
    const int tok = blockIdx.x, sq = blockIdx.y;
    const int c = (blockIdx.z * SC_THREADS + threadIdx.x) * V;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    if (slot < 0 || slot >= n_slots || tok >= n_new || c >= E) return;
    T* tl = tail + (size_t)slot * (taps - 1) * E + c;
    const T* hr = h + (size_t)row0 * E + c;
    float own[V], acc[V], v[V];
    load_values<T, V>(hr + (size_t)tok * E, own);
#pragma unroll
    for (int k = 0; k < V; k++) acc[k] = 0.0f;
    for (int j = 0; j < taps; j++) {
        const int back = taps - 1 - j;
        // The input `back` positions earlier: a row of this step, or one the tail kept.
        if (back == 0) {
#pragma unroll
            for (int k = 0; k < V; k++) v[k] = own[k];
        } else if (back <= tok) {
            load_values<T, V>(hr + (size_t)(tok - back) * E, v);
        } else {
            load_values<T, V>(tl + (size_t)(tok - back + taps - 1) * E, v);
        }
#pragma unroll
        for (int k = 0; k < V; k++) acc[k] = fmaf(w[(size_t)j * E + c + k], v[k], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < V; k++) acc[k] += own[k];
    store_values<T, V>(out + (size_t)(row0 + tok) * E + c, acc);
    if (update_tail) {
        // One row a sequence: the tail moves up by one and takes this row's input.
        for (int i = 0; i + 2 < taps; i++) {
            load_values<T, V>(tl + (size_t)(i + 1) * E, v);
            store_values<T, V>(tl + (size_t)i * E, v);
        }
        if (taps > 1) store_values<T, V>(tl + (size_t)(taps - 2) * E, own);
    }
}

// The same sums for prompts: a thread walks SC_ROWS rows of one sequence for its V channels with the last
// TAPS - 1 inputs and the kernel in registers, so that every input is read once.
#define SC_ROWS 8
template <class T, int V, int TAPS>
__global__ void __launch_bounds__(SC_THREADS)
short_conv_rows_kernel(const T* __restrict__ h, const float* __restrict__ w, const T* __restrict__ tail, const int* __restrict__ seq_rows,
                       const int* __restrict__ seq_slot, T* __restrict__ out, int E, int n_slots) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(h); PDL_FRESH(tail);
    const int tok0 = blockIdx.x * SC_ROWS, sq = blockIdx.y;
    const int c = (blockIdx.z * SC_THREADS + threadIdx.x) * V;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    if (slot < 0 || slot >= n_slots || tok0 >= n_new || c >= E) return;
    const T* tl = tail + (size_t)slot * (TAPS - 1) * E + c;
    const T* hr = h + (size_t)row0 * E + c;
    float wt[TAPS][V], win[TAPS - 1][V], own[V], acc[V];
#pragma unroll
    for (int j = 0; j < TAPS; j++)
#pragma unroll
        for (int k = 0; k < V; k++) wt[j][k] = w[(size_t)j * E + c + k];
#pragma unroll
    for (int i = 0; i < TAPS - 1; i++) {       // the input at row tok0 - (TAPS - 1) + i of the step, or what the tail kept of it
        const int rel = tok0 - (TAPS - 1) + i;
        if (rel >= 0) load_values<T, V>(hr + (size_t)rel * E, win[i]);
        else load_values<T, V>(tl + (size_t)(rel + TAPS - 1) * E, win[i]);
    }
    const int n = min(SC_ROWS, n_new - tok0);
    for (int t = 0; t < n; t++) {
        load_values<T, V>(hr + (size_t)(tok0 + t) * E, own);
#pragma unroll
        for (int k = 0; k < V; k++) {
            float a = 0.0f;
#pragma unroll
            for (int j = 0; j < TAPS - 1; j++) a = fmaf(wt[j][k], win[j][k], a);
            acc[k] = own[k] + fmaf(wt[TAPS - 1][k], own[k], a);
        }
        store_values<T, V>(out + (size_t)(row0 + tok0 + t) * E + c, acc);
#pragma unroll
        for (int i = 0; i + 1 < TAPS - 1; i++)
#pragma unroll
            for (int k = 0; k < V; k++) win[i][k] = win[i + 1][k];
#pragma unroll
        for (int k = 0; k < V; k++) win[TAPS - 2][k] = own[k];
    }
}

// The tail after the step: the inputs at the last taps - 1 positions the sequence now holds,
// from this step's rows where they reach that far back, else from the old tail (entry i takes
// old entry i + n_new, which lies above it, so ascending i never reads what it has written).
template <class T>
__global__ void __launch_bounds__(SC_THREADS)
short_conv_tail_kernel(const T* __restrict__ h, T* __restrict__ tail, const int* __restrict__ seq_rows, const int* __restrict__ seq_slot,
                       int E, int taps, int n_slots) {
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(h);
    const int sq = blockIdx.x;
    const int c = blockIdx.y * SC_THREADS + threadIdx.x;
    const int slot = seq_slot[sq];
    const int row0 = seq_rows[sq], n_new = seq_rows[sq + 1] - row0;
    if (slot < 0 || slot >= n_slots || n_new <= 0 || c >= E) return;
    T* tl = tail + (size_t)slot * (taps - 1) * E + c;
    for (int i = 0; i < taps - 1; i++) {
        const int rel = n_new - (taps - 1) + i;      // which row of this step, if not negative
        tl[(size_t)i * E] = rel >= 0 ? h[(size_t)(row0 + rel) * E + c] : tl[(size_t)(i + n_new) * E];
    }
}

// Two RMS norms of the same row share its statistic: out1 = x / rms(x) * w1, out2 = x / rms(x) * w2
// (out2 may be null).  With `taps` > 0 the first output also passes the convolution above, for steps of one
// row a sequence only (row r is sequence r's one row): the sum runs over the tail and the row's own rounded
// value in the same order as in short_conv_kernel, so both ways give the same bits; the tail moves up by one.
template <class T>
__global__ void __launch_bounds__(1024)
norm_pair_conv_kernel(const float* __restrict__ x, const float* __restrict__ w1, const float* __restrict__ w2, const float* __restrict__ cw,
                      T* __restrict__ tail, const int* __restrict__ row_slot, T* __restrict__ out1, T* __restrict__ out2, int E, float eps,
                      int taps, int n_slots, int update_tail) {
    __shared__ float scratch[32];
    pdl_launch_dependents_if_resident();
    pdl_wait();
    PDL_FRESH(x);
    const int r = blockIdx.x;
    const float* xr = x + (size_t)r * E;
    // A thread takes four neighbouring channels at a time where the width allows (W = 4), else one: which values it
    // adds up and in which order depends on the width alone.
    const int W = E % 4 == 0 ? 4 : 1;
    float ss = 0.0f;
    if (W == 4) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
    } else {
        for (int c = threadIdx.x; c < E; c += blockDim.x) ss += xr[c] * xr[c];
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)E + eps);
    const int slot = taps > 0 ? row_slot[r] : -1;
    const bool conv = taps > 0 && slot >= 0 && slot < n_slots;
    if (W == 4 && !conv) {
        for (int c = 4 * threadIdx.x; c < E; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + c);
            const float4 g = *reinterpret_cast<const float4*>(w1 + c);
            const float o1[4] = {v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w};
            store_values<T, 4>(out1 + (size_t)r * E + c, o1);
            if (out2) {
                const float4 g2 = *reinterpret_cast<const float4*>(w2 + c);
                const float o2[4] = {v.x * scale * g2.x, v.y * scale * g2.y, v.z * scale * g2.z, v.w * scale * g2.w};
                store_values<T, 4>(out2 + (size_t)r * E + c, o2);
            }
        }
        return;
    }
    for (int c0 = W * threadIdx.x; c0 < E; c0 += W * blockDim.x) {
        for (int c = c0; c < c0 + W; c++) {
            const float v = xr[c];
            const T h = from_f32<T>(v * scale * w1[c]);
            if (out2) out2[(size_t)r * E + c] = from_f32<T>(v * scale * w2[c]);
            if (!conv) {
                out1[(size_t)r * E + c] = h;
                continue;
            }
            T* tl = tail + (size_t)slot * (taps - 1) * E + c;
            const float own = to_f32(h);
            float acc = 0.0f;
            for (int j = 0; j + 1 < taps; j++) acc = fmaf(cw[(size_t)j * E + c], to_f32(tl[(size_t)j * E]), acc);
            acc = fmaf(cw[(size_t)(taps - 1) * E + c], own, acc);
            out1[(size_t)r * E + c] = from_f32<T>(own + acc);
            if (update_tail) {
                for (int i = 0; i + 2 < taps; i++) tl[(size_t)i * E] = tl[(size_t)(i + 1) * E];
                if (taps > 1) tl[(size_t)(taps - 2) * E] = h;
            }
        }
    }
}

template <class T>
static int launch_pair(const float* x, const float* w1, const float* w2, const float* cw, void* tail, const int* row_slot, void* out1,
                       void* out2, int rows, int E, float eps, int taps, int n_slots, int update_tail, cudaStream_t s) {
    BC_CHECK_ARG(rows >= 0 && E > 0 && taps >= 0, "norm_pair: bad sizes rows=%d E=%d taps=%d", rows, E, taps);
    BC_CHECK_ARG(taps == 0 || (cw && row_slot && (tail || taps == 1)), "norm_pair: the convolution needs its weights, the rows' slots and the tail");
    if (rows == 0) return BC_OK;
    // The block's size depends on the row's width alone, never on the number of rows: a row's statistic is the same bits in any batch.
    const int threads = E >= 8192 ? 1024 : E >= 2048 ? 512 : 256;
    bc_launch(norm_pair_conv_kernel<T>, dim3(rows), dim3(threads), 0, s, x, w1, w2, cw, (T*)tail, row_slot, (T*)out1, (T*)out2, E, eps, taps,
              n_slots, update_tail);
    BC_LAUNCH_STATUS();
}

// x: [rows, E] float; w1, w2: [E] float; out1, out2: [rows, E] (out2 and w2 may be null).  taps 0: no convolution;
// else cw [taps, E], tail [n_slots, taps - 1, E], row_slot [rows], every row being its sequence's only row of the step.
extern "C" int bc_norm_pair_f32(const float* x, const float* w1, const float* w2, const float* cw, void* tail, const int* row_slot, void* out1,
                                void* out2, int rows, int E, float eps, int taps, int n_slots, int update_tail, cudaStream_t s) {
    return launch_pair<float>(x, w1, w2, cw, tail, row_slot, out1, out2, rows, E, eps, taps, n_slots, update_tail, s);
}
extern "C" int bc_norm_pair_bf16(const float* x, const float* w1, const float* w2, const float* cw, void* tail, const int* row_slot, void* out1,
                                 void* out2, int rows, int E, float eps, int taps, int n_slots, int update_tail, cudaStream_t s) {
    return launch_pair<bf16>(x, w1, w2, cw, tail, row_slot, out1, out2, rows, E, eps, taps, n_slots, update_tail, s);
}

template <class T>
static int launch(const void* h, const float* w, void* tail, const int* seq_rows, const int* seq_slot, void* out, int seqs, int max_new,
                  int E, int taps, int n_slots, int write_tail, cudaStream_t s) {
    BC_CHECK_ARG(seqs >= 0 && seqs <= 65535 && max_new >= 0 && E > 0 && taps >= 1, "short_conv: bad sizes seqs=%d max_new=%d E=%d taps=%d",
                 seqs, max_new, E, taps);
    BC_CHECK_ARG((E + SC_THREADS - 1) / SC_THREADS <= 65535, "short_conv: %d channels are too many", E);
    if (seqs == 0 || max_new == 0) return BC_OK;
    const int chunks = (E + SC_THREADS - 1) / SC_THREADS;
    const int fused = write_tail && max_new == 1;
    constexpr int V = 16 / (int)sizeof(T);
    const bool wide = E % V == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)tail % 16 == 0;
    const dim3 rows_grid((max_new + SC_ROWS - 1) / SC_ROWS, seqs, (E / V + SC_THREADS - 1) / SC_THREADS);
#define SC_CASE(TAPS)                                                                                                                   \
    case TAPS:                                                                                                                          \
        bc_launch(short_conv_rows_kernel<T, V, TAPS>, rows_grid, dim3(SC_THREADS), 0, s, (const T*)h, w, (const T*)tail, seq_rows, seq_slot, \
                  (T*)out, E, n_slots);                                                                                                 \
        break;
    if (wide && max_new > 1 && taps >= 2 && taps <= 8) {
        switch (taps) { SC_CASE(2) SC_CASE(3) SC_CASE(4) SC_CASE(5) SC_CASE(6) SC_CASE(7) SC_CASE(8) }
    } else if (wide)
        bc_launch(short_conv_kernel<T, V>, dim3(max_new, seqs, (E / V + SC_THREADS - 1) / SC_THREADS), dim3(SC_THREADS), 0, s, (const T*)h, w,
                  (T*)tail, seq_rows, seq_slot, (T*)out, E, taps, n_slots, fused);
    else
        bc_launch(short_conv_kernel<T, 1>, dim3(max_new, seqs, chunks), dim3(SC_THREADS), 0, s, (const T*)h, w, (T*)tail, seq_rows, seq_slot,
                  (T*)out, E, taps, n_slots, fused);
#undef SC_CASE
    if (write_tail && !fused && taps > 1) {
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            bc_set_error("short_conv: %s", cudaGetErrorString(e));
            return (int)e;
        }
        bc_launch(short_conv_tail_kernel<T>, dim3(seqs, chunks), dim3(SC_THREADS), 0, s, (const T*)h, (T*)tail, seq_rows, seq_slot, E, taps,
                  n_slots);
    }
    BC_LAUNCH_STATUS();
}

// h, out: [rows, E]; w: [taps, E] float (tap by tap, so that neighbouring channels are neighbours); tail: [n_slots, taps - 1, E].  Sequence s owns rows
// seq_rows[s] .. seq_rows[s + 1] and lives in slot seq_slot[s] (negative: skipped, its rows of
// `out` are left untouched).  max_new: the most rows any sequence brings.  write_tail 0 leaves
// the tail as it was (a run that reads another run's memory).
extern "C" int bc_short_conv_f32(const void* h, const float* w, void* tail, const int* seq_rows, const int* seq_slot, void* out, int seqs,
                                 int max_new, int E, int taps, int n_slots, int write_tail, cudaStream_t s) {
    return launch<float>(h, w, tail, seq_rows, seq_slot, out, seqs, max_new, E, taps, n_slots, write_tail, s);
}
extern "C" int bc_short_conv_bf16(const void* h, const float* w, void* tail, const int* seq_rows, const int* seq_slot, void* out, int seqs,
                                  int max_new, int E, int taps, int n_slots, int write_tail, cudaStream_t s) {
    return launch<bf16>(h, w, tail, seq_rows, seq_slot, out, seqs, max_new, E, taps, n_slots, write_tail, s);
}
