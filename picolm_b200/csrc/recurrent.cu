// Kernels of the mixers that carry a fixed-size state from token to token, and of the small steps around
// them, for ragged steps (every sequence brings its own number of tokens, one in a decode step):
//
//   plm_causal_conv        depthwise causal convolution over the tokens of each sequence + SiLU, the last
//                          taps - 1 inputs of each sequence kept as state
//   plm_linear_scan        S_t = diag(d_t) S_(t-1) + k_t v_t^T, y_t = S_t^T q_t (+ skip * v_t): the recurrence
//                          of gated linear attention and of state-space duality, the decay per key channel
//                          or per head, computed from the raw projections inside the kernel in fp32
//   plm_gated_norm         grouped RMS norm with a multiplicative gate before or after it (or only one of the two)
//   plm_head_linear        out[t, h, :] = W[h] x[t, h, :]: one small matrix per head
//   plm_store_rows_paged   rows of the step's tokens into the pages of a cache
//
// Everything that enters a recurrence is fp32: decays, step sizes, the state, the sums.  T is the run's
// element type (float or bf16) of projections and activations; small parameter vectors are fp32.
#include "common.cuh"

#define SCAN_THREADS 128
#define SCAN_PTILE 32

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// ------------------------------------------------------------------------------------------------ convolution
// u [T, C] with row stride ldu; w [C, taps], the last tap being the current token's; state [slot][taps - 1][C],
// oldest first.  One thread per (token, channel): inputs before the step's first token come from the state.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ u, long ldu, const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, long state_stride, const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, T* __restrict__ out,
                                   int n_tokens, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * C) return;
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int b = PLM_SEQ_NO(tok_seq[t]);
    const int i = t - seq_start[b];
    const float* st = state + (long)seq_slot[b] * state_stride;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j, li = i - back;
        const float val = li >= 0 ? to_f32<T>(u[(long)(t - back) * ldu + c]) : st[(long)(taps - 1 + li) * C + c];
        acc = fmaf(w[(long)c * taps + j], val, acc);
    }
    out[(long)t * C + c] = from_f32<T>(silu_f(acc));
}

// The state after the step: the last taps - 1 inputs of old state followed by the step's tokens.  One thread per
// (sequence, channel); it reads what it needs of the old state before it writes.
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ u, long ldu, float* __restrict__ state, long state_stride,
                                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int n_seqs,
                                         int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
    float* st = state + (long)seq_slot[b] * state_stride;
    // ascending s: slot s takes old slot s + n (> s), which no earlier iteration has overwritten
    for (int s = 0; s < taps - 1; ++s) {
        const int src = n - (taps - 1) + s;
        st[(long)s * C + c] = src >= 0 ? to_f32<T>(u[(long)(t0 + src) * ldu + c]) : st[(long)(s + n) * C + c];
    }
}

// A decode step (one token per sequence): output and new state by the same thread.
template <typename T>
__global__ void causal_conv_decode_kernel(const T* __restrict__ u, long ldu, const float* __restrict__ w,
                                          const float* __restrict__ bias, float* __restrict__ state, long state_stride,
                                          const int* __restrict__ seq_slot, T* __restrict__ out, int n_seqs, int C, int taps) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int b = (int)(idx / C), c = (int)(idx % C);
    float* st = state + (long)seq_slot[b] * state_stride;
    const float cur = to_f32<T>(u[(long)b * ldu + c]);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps - 1; ++j) {
        const float val = st[(long)j * C + c];
        acc = fmaf(w[(long)c * taps + j], val, acc);
        if (j > 0) st[(long)(j - 1) * C + c] = val;
    }
    acc = fmaf(w[(long)c * taps + taps - 1], cur, acc);
    if (taps > 1) st[(long)(taps - 2) * C + c] = cur;
    out[(long)b * C + c] = from_f32<T>(silu_f(acc));
}

extern "C" int plm_causal_conv(const void* u, int dtype, long ldu, const float* w, const float* bias, float* state,
                               long state_stride, const int* tok_seq, const int* seq_start, const int* seq_slot, void* out,
                               int n_tokens, int n_seqs, int C, int taps, int is_decode, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0 || C <= 0 || taps < 1) return PLM_ERR_SHAPE;
    if (dtype != PLM_F32 && dtype != PLM_BF16) return PLM_ERR_DTYPE;
    const int nt = 256;
    cudaError_t e;
    if (is_decode) {
        const unsigned grid = (unsigned)(((long)n_seqs * C + nt - 1) / nt);
        e = dtype == PLM_F32
                ? launch_pdl(causal_conv_decode_kernel<float>, dim3(grid), dim3(nt), 0, stream, (const float*)u, ldu, w, bias, state,
                             state_stride, seq_slot, (float*)out, n_seqs, C, taps)
                : launch_pdl(causal_conv_decode_kernel<bf16>, dim3(grid), dim3(nt), 0, stream, (const bf16*)u, ldu, w, bias, state,
                             state_stride, seq_slot, (bf16*)out, n_seqs, C, taps);
        return plm_status_of(e);
    }
    const unsigned grid = (unsigned)(((long)n_tokens * C + nt - 1) / nt);
    e = dtype == PLM_F32
            ? launch_pdl(causal_conv_kernel<float>, dim3(grid), dim3(nt), 0, stream, (const float*)u, ldu, w, bias, (const float*)state,
                         state_stride, tok_seq, seq_start, seq_slot, (float*)out, n_tokens, C, taps)
            : launch_pdl(causal_conv_kernel<bf16>, dim3(grid), dim3(nt), 0, stream, (const bf16*)u, ldu, w, bias, (const float*)state,
                         state_stride, tok_seq, seq_start, seq_slot, (bf16*)out, n_tokens, C, taps);
    if (e != cudaSuccess) return (int)e;
    if (taps == 1) return PLM_OK;
    const unsigned grid2 = (unsigned)(((long)n_seqs * C + nt - 1) / nt);
    e = dtype == PLM_F32
            ? launch_pdl(causal_conv_state_kernel<float>, dim3(grid2), dim3(nt), 0, stream, (const float*)u, ldu, state, state_stride,
                         seq_start, seq_slot, n_seqs, C, taps)
            : launch_pdl(causal_conv_state_kernel<bf16>, dim3(grid2), dim3(nt), 0, stream, (const bf16*)u, ldu, state, state_stride,
                         seq_start, seq_slot, n_seqs, C, taps);
    return plm_status_of(e);
}

// ------------------------------------------------------------------------------------------------ the scan
// How the decay d_t and the scale of v_t come out of the raw projections (all in fp32):
//   DECAY_STEP     per head: dt = softplus(raw[t, h] + p0[h]); d = exp(-exp(p1[h]) * dt); v_t is scaled by dt
//   DECAY_SIGMOID  per key channel: d[n] = exp(log_sigmoid(raw[t, h * N + n] + p0[h * N + n]) * power)
#define DECAY_STEP 1
#define DECAY_SIGMOID 2

struct ScanArgs {
    const void *q, *k, *v, *raw;          // [T, groups * N], [T, groups * N], [T, H * P], the decay's raw values
    long ldq, ldk, ldv, ldraw;            // row strides in elements
    const float *p0, *p1, *skip;          // see the decay modes; skip[h] (or null): y += skip[h] * v_t (the unscaled v)
    float q_scale, power;
    float* state;                         // [slot][H][N][P]
    long state_stride;
    float* y;                             // [T, H * P]
    long ldy;
    const int *seq_start, *seq_slot;
    int n_seqs, H, N, P, heads_per_group;
};

// One block per (sequence, head, tile of 32 value columns).  A warp holds 8 columns; the N rows of a column's
// state are dealt to 4 lanes (NS consecutive rows each, in registers).  The tokens of the sequence are taken in
// order, TC at a time: the block first brings their q, k, decay and v to shared memory as fp32 (the
// exponentials are taken there, once per token and channel), then every thread steps its rows through them.
template <typename T, int NS, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(const ScanArgs a, int TC) {
    constexpr int ROW = NS + 4;                           // padded so that the four lanes' float4 reads hit different banks
    constexpr bool PER_CHANNEL = MODE == DECAY_SIGMOID;
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    int bid = blockIdx.x;
    const int ptile = bid % ptiles;
    bid /= ptiles;
    const int h = bid % a.H, b = bid / a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npart = lane >> 3, pl = (warp << 3) + (lane & 7);
    const int p = ptile * SCAN_PTILE + pl;
    const int g = h / a.heads_per_group;
    const int N = a.N, P = a.P;
    float* qs = smem;                                     // [TC][4][ROW]
    float* ks = qs + (long)TC * 4 * ROW;
    float* ds = ks + (long)TC * 4 * ROW;                  // per channel: [TC][4][ROW]; per head: [TC] decay, [TC] scale of v
    float* vs = ds + (PER_CHANNEL ? (long)TC * 4 * ROW : 2L * TC);    // [TC][SCAN_PTILE]
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    const T* raw = (const T*)a.raw;
    pdl_wait();
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    float* st = a.state + (long)a.seq_slot[b] * a.state_stride + (long)h * N * P;
    float S[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = npart * NS + i;
        S[i] = (n < N && p < P) ? st[(long)n * P + p] : 0.f;
    }
    const float skip = a.skip ? a.skip[h] : 0.f;
    for (int base = t0; base < t1; base += TC) {
        const int nt = min(TC, t1 - base);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * 4 * NS; idx += SCAN_THREADS) {
            const int tt = idx / (4 * NS), n = idx % (4 * NS);
            const int at = (tt * 4 + n / NS) * ROW + n % NS;
            const long row = base + tt;
            const bool in = n < N;
            qs[at] = in ? to_f32<T>(q[row * a.ldq + (long)g * N + n]) * a.q_scale : 0.f;
            ks[at] = in ? to_f32<T>(k[row * a.ldk + (long)g * N + n]) : 0.f;
            if (PER_CHANNEL)
                ds[at] = in ? expf(log_sigmoid_f(to_f32<T>(raw[row * a.ldraw + (long)h * N + n]) + a.p0[(long)h * N + n]) * a.power) : 0.f;
        }
        if (!PER_CHANNEL) {
            for (int tt = threadIdx.x; tt < nt; tt += SCAN_THREADS) {
                const float dt = softplus_f(to_f32<T>(raw[(long)(base + tt) * a.ldraw + h]) + a.p0[h]);
                ds[tt] = expf(-expf(a.p1[h]) * dt);
                ds[TC + tt] = dt;
            }
        }
        for (int idx = threadIdx.x; idx < nt * SCAN_PTILE; idx += SCAN_THREADS) {
            const int tt = idx / SCAN_PTILE, c = idx % SCAN_PTILE, pc = ptile * SCAN_PTILE + c;
            vs[idx] = pc < P ? to_f32<T>(v[(long)(base + tt) * a.ldv + (long)h * P + pc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float x = vs[tt * SCAN_PTILE + pl];
            const float vv = PER_CHANNEL ? x : ds[TC + tt] * x;
            const float dh = PER_CHANNEL ? 0.f : ds[tt];
            const float4* q4 = (const float4*)(qs + (tt * 4 + npart) * ROW);
            const float4* k4 = (const float4*)(ks + (tt * 4 + npart) * ROW);
            const float4* d4 = (const float4*)(ds + (tt * 4 + npart) * ROW);
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < NS / 4; ++i) {
                const float4 qq = q4[i], kk = k4[i];
                float4 dd;
                if (PER_CHANNEL) dd = d4[i];
                else dd = make_float4(dh, dh, dh, dh);
                S[4 * i + 0] = fmaf(dd.x, S[4 * i + 0], kk.x * vv);
                S[4 * i + 1] = fmaf(dd.y, S[4 * i + 1], kk.y * vv);
                S[4 * i + 2] = fmaf(dd.z, S[4 * i + 2], kk.z * vv);
                S[4 * i + 3] = fmaf(dd.w, S[4 * i + 3], kk.w * vv);
                acc0 = fmaf(S[4 * i + 0], qq.x, acc0);
                acc1 = fmaf(S[4 * i + 1], qq.y, acc1);
                acc0 = fmaf(S[4 * i + 2], qq.z, acc0);
                acc1 = fmaf(S[4 * i + 3], qq.w, acc1);
            }
            float acc = acc0 + acc1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (npart == 0 && p < P) a.y[(long)(base + tt) * a.ldy + (long)h * P + p] = fmaf(skip, x, acc);
        }
    }
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = npart * NS + i;
        if (n < N && p < P) st[(long)n * P + p] = S[i];
    }
}

template <typename T, int NS>
static cudaError_t scan_launch(const ScanArgs& a, int mode, cudaStream_t stream) {
    const int ROW = NS + 4;
    // tokens per pass: as many as fit into about 36 KB of shared memory, 16 at most
    const long per_token = (mode == DECAY_SIGMOID ? 3L : 2L) * 4 * ROW + SCAN_PTILE + 2;
    int TC = (int)((36 * 1024 / 4) / per_token);
    TC = TC > 16 ? 16 : TC < 1 ? 1 : TC;
    const size_t smem = (size_t)(per_token * TC) * sizeof(float);
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    const dim3 grid((unsigned)((long)a.n_seqs * a.H * ptiles));
    if (mode == DECAY_SIGMOID)
        return launch_pdl(linear_scan_kernel<T, NS, DECAY_SIGMOID>, grid, dim3(SCAN_THREADS), smem, stream, a, TC);
    return launch_pdl(linear_scan_kernel<T, NS, DECAY_STEP>, grid, dim3(SCAN_THREADS), smem, stream, a, TC);
}

template <typename T>
static int scan_dispatch(const ScanArgs& a, int mode, cudaStream_t stream) {
    const int ns = (a.N + 3) / 4;
    cudaError_t e;
    if (ns <= 4) e = scan_launch<T, 4>(a, mode, stream);
    else if (ns <= 8) e = scan_launch<T, 8>(a, mode, stream);
    else if (ns <= 16) e = scan_launch<T, 16>(a, mode, stream);
    else if (ns <= 32) e = scan_launch<T, 32>(a, mode, stream);
    else if (ns <= 64) e = scan_launch<T, 64>(a, mode, stream);
    else return PLM_ERR_UNSUPPORTED;
    return plm_status_of(e);
}

extern "C" int plm_linear_scan(const void* q, const void* k, const void* v, const void* raw, int dtype, long ldq, long ldk,
                               long ldv, long ldraw, int mode, const float* p0, const float* p1, const float* skip,
                               float q_scale, float power, float* state, long state_stride, float* y, long ldy,
                               const int* seq_start, const int* seq_slot, int n_seqs, int H, int N, int P,
                               int heads_per_group, cudaStream_t stream) {
    if (n_seqs <= 0 || H <= 0 || N <= 0 || P <= 0 || heads_per_group <= 0) return PLM_ERR_SHAPE;
    if (mode != DECAY_STEP && mode != DECAY_SIGMOID) return PLM_ERR_UNSUPPORTED;
    if (mode == DECAY_STEP && !p1) return PLM_ERR_SHAPE;
    if (!p0) return PLM_ERR_SHAPE;
    if (N > 256) return PLM_ERR_UNSUPPORTED;
    ScanArgs a;
    a.q = q, a.k = k, a.v = v, a.raw = raw;
    a.ldq = ldq, a.ldk = ldk, a.ldv = ldv, a.ldraw = ldraw;
    a.p0 = p0, a.p1 = p1, a.skip = skip;
    a.q_scale = q_scale, a.power = power;
    a.state = state, a.state_stride = state_stride;
    a.y = y, a.ldy = ldy;
    a.seq_start = seq_start, a.seq_slot = seq_slot;
    a.n_seqs = n_seqs, a.H = H, a.N = N, a.P = P, a.heads_per_group = heads_per_group;
    if (dtype == PLM_F32) return scan_dispatch<float>(a, mode, stream);
    if (dtype == PLM_BF16) return scan_dispatch<bf16>(a, mode, stream);
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ gate and norm
// One warp per (row, group of `group` consecutive columns):
//   val = x * act(gate)                       (gate_mode 1: the gate comes before the norm)
//   val = val / sqrt(mean(val^2) + eps) * w   (do_norm; w indexed by the column, or by the column within its group)
//   val = val * act(gate)                     (gate_mode 2: the gate comes after the norm)
// act: 0 SiLU, 1 sigmoid.  Statistics and products in fp32.
template <typename TI, typename TG, typename TO>
__global__ void gated_norm_kernel(const TI* __restrict__ x, long ldx, const TG* __restrict__ gate, long ldg,
                                  const float* __restrict__ w, int w_per_group, TO* __restrict__ out, long ldo, int n_rows,
                                  int C, int group, float eps, int gate_mode, int act, int do_norm) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = C / group;
    const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long)n_rows * groups) return;
    const long t = wid / groups;
    const int c0 = (int)(wid % groups) * group;
    const TI* xr = x + t * ldx + c0;
    const TG* gr = gate ? gate + t * ldg + c0 : nullptr;
    float r = 1.f;
    if (do_norm) {
        float ss = 0.f;
        for (int c = lane; c < group; c += 32) {
            float val = to_f32<TI>(xr[c]);
            if (gate_mode == 1) {
                const float gg = to_f32<TG>(gr[c]);
                val *= act ? sigmoid_f(gg) : silu_f(gg);
            }
            ss = fmaf(val, val, ss);
        }
        ss = warp_sum(ss);
        r = 1.f / sqrtf(ss / (float)group + eps);
    }
    for (int c = lane; c < group; c += 32) {
        float val = to_f32<TI>(xr[c]);
        float ga = 1.f;
        if (gate_mode) {
            const float gg = to_f32<TG>(gr[c]);
            ga = act ? sigmoid_f(gg) : silu_f(gg);
        }
        if (gate_mode == 1) val *= ga;
        if (do_norm) {
            val *= r;
            if (w) val *= w[w_per_group ? c : c0 + c];
        }
        if (gate_mode == 2) val *= ga;
        out[t * ldo + c0 + c] = from_f32<TO>(val);
    }
}

template <typename TI, typename TG, typename TO>
static int gated_norm_launch(const void* x, long ldx, const void* gate, long ldg, const float* w, int w_per_group, void* out,
                             long ldo, int n_rows, int C, int group, float eps, int gate_mode, int act, int do_norm,
                             cudaStream_t stream) {
    const long warps = (long)n_rows * (C / group);
    const unsigned grid = (unsigned)((warps * 32 + 255) / 256);
    return plm_status_of(launch_pdl(gated_norm_kernel<TI, TG, TO>, dim3(grid), dim3(256), 0, stream, (const TI*)x, ldx,
                                    (const TG*)gate, ldg, w, w_per_group, (TO*)out, ldo, n_rows, C, group, eps, gate_mode, act,
                                    do_norm));
}

extern "C" int plm_gated_norm(const void* x, int x_dtype, long ldx, const void* gate, int gate_dtype, long ldg, const float* w,
                              int w_per_group, void* out, int out_dtype, long ldo, int n_rows, int C, int group, float eps,
                              int gate_mode, int act, int do_norm, cudaStream_t stream) {
    if (n_rows <= 0 || C <= 0 || group <= 0 || C % group) return PLM_ERR_SHAPE;
    if (gate_mode && !gate) return PLM_ERR_SHAPE;
    if (!gate) gate_dtype = PLM_BF16;
    const int key = (x_dtype << 2) | (gate_dtype << 1) | out_dtype;
#define GN(TI, TG, TO) \
    return gated_norm_launch<TI, TG, TO>(x, ldx, gate, ldg, w, w_per_group, out, ldo, n_rows, C, group, eps, gate_mode, act, do_norm, stream)
    switch (key) {
        case (PLM_F32 << 2) | (PLM_F32 << 1) | PLM_F32: GN(float, float, float);
        case (PLM_F32 << 2) | (PLM_F32 << 1) | PLM_BF16: GN(float, float, bf16);
        case (PLM_F32 << 2) | (PLM_BF16 << 1) | PLM_F32: GN(float, bf16, float);
        case (PLM_F32 << 2) | (PLM_BF16 << 1) | PLM_BF16: GN(float, bf16, bf16);
        case (PLM_BF16 << 2) | (PLM_F32 << 1) | PLM_F32: GN(bf16, float, float);
        case (PLM_BF16 << 2) | (PLM_F32 << 1) | PLM_BF16: GN(bf16, float, bf16);
        case (PLM_BF16 << 2) | (PLM_BF16 << 1) | PLM_F32: GN(bf16, bf16, float);
        case (PLM_BF16 << 2) | (PLM_BF16 << 1) | PLM_BF16: GN(bf16, bf16, bf16);
    }
#undef GN
    return PLM_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------------ one matrix per head
// out[t, h, o] = sum_i W[h][o][i] * x[t, h, i], optionally times sigmoid(gate[t, h, o]).  x [T, H * I] with row stride
// ldx, W [H, O, I], out [T, H * O].  Tiles of 16 tokens x 64 outputs, the inputs walked 32 at a time through shared
// memory, sums in fp32 in ascending order of i.
#define HL_TT 16
#define HL_TO 64
#define HL_TI 32
template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ W,
                                                          const T* __restrict__ gate, long ldg, T* __restrict__ out, long ldo,
                                                          int n_tokens, int H, int O, int I) {
    __shared__ float xs[HL_TT][HL_TI + 1];
    __shared__ float ws[HL_TO][HL_TI + 1];
    pdl_launch_dependents();
    const int h = blockIdx.z, t0 = blockIdx.y * HL_TT, o0 = blockIdx.x * HL_TO;
    const int ol = threadIdx.x % HL_TO, tg = threadIdx.x / HL_TO;          // 4 token groups of 4 tokens each
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    pdl_wait();
    for (int i0 = 0; i0 < I; i0 += HL_TI) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < HL_TT * HL_TI; idx += 256) {
            const int tt = idx / HL_TI, ii = idx % HL_TI;
            xs[tt][ii] = (t0 + tt < n_tokens && i0 + ii < I) ? to_f32<T>(x[(long)(t0 + tt) * ldx + (long)h * I + i0 + ii]) : 0.f;
        }
        for (int idx = threadIdx.x; idx < HL_TO * HL_TI; idx += 256) {
            const int oo = idx / HL_TI, ii = idx % HL_TI;
            ws[oo][ii] = (o0 + oo < O && i0 + ii < I) ? to_f32<T>(W[((long)h * O + o0 + oo) * I + i0 + ii]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int ii = 0; ii < HL_TI; ++ii) {
            const float wv = ws[ol][ii];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(wv, xs[tg * 4 + j][ii], acc[j]);
        }
    }
    if (o0 + ol < O) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = t0 + tg * 4 + j;
            if (t < n_tokens) {
                float val = acc[j];
                if (gate) val *= sigmoid_f(to_f32<T>(gate[(long)t * ldg + (long)h * O + o0 + ol]));
                out[(long)t * ldo + (long)h * O + o0 + ol] = from_f32<T>(val);
            }
        }
    }
}

extern "C" int plm_head_linear(const void* x, int dtype, long ldx, const void* W, const void* gate, long ldg, void* out, long ldo,
                               int n_tokens, int H, int O, int I, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || O <= 0 || I <= 0 || H > 65535) return PLM_ERR_SHAPE;
    const dim3 grid((O + HL_TO - 1) / HL_TO, (n_tokens + HL_TT - 1) / HL_TT, H);
    if (grid.y > 65535) return PLM_ERR_SHAPE;
    cudaError_t e;
    if (dtype == PLM_F32)
        e = launch_pdl(head_linear_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ldx, (const float*)W, (const float*)gate,
                       ldg, (float*)out, ldo, n_tokens, H, O, I);
    else if (dtype == PLM_BF16)
        e = launch_pdl(head_linear_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, (const bf16*)W, (const bf16*)gate,
                       ldg, (bf16*)out, ldo, n_tokens, H, O, I);
    else
        return PLM_ERR_DTYPE;
    return plm_status_of(e);
}

// ------------------------------------------------------------------------------------------------ rows into pages
// pages [n_pages][PLM_PAGE][R] (one kv head): row t goes to position tok_pos[t] of sequence tok_seq[t].
template <typename T>
__global__ void store_rows_paged_kernel(const T* __restrict__ rows, long ld, T* __restrict__ pages, const int* __restrict__ tok_pos,
                                        const int* __restrict__ tok_seq, const int* __restrict__ block_table, int pages_per_seq,
                                        int n_tokens, int R) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * R) return;
    const int t = (int)(idx / R), c = (int)(idx % R);
    const int pos = PLM_POSITION(tok_pos[t]);
    const int page = PLM_PAGE_NO(block_table[(long)PLM_SEQ_NO(tok_seq[t]) * pages_per_seq + pos / PLM_PAGE]);
    pages[((long)page * PLM_PAGE + pos % PLM_PAGE) * R + c] = rows[(long)t * ld + c];
}

extern "C" int plm_store_rows_paged(const void* rows, int dtype, long ld, void* pages, const int* tok_pos, const int* tok_seq,
                                    const int* block_table, int pages_per_seq, int n_tokens, int R, cudaStream_t stream) {
    if (n_tokens <= 0 || R <= 0) return PLM_ERR_SHAPE;
    const unsigned grid = (unsigned)(((long)n_tokens * R + 255) / 256);
    cudaError_t e;
    if (dtype == PLM_F32)
        e = launch_pdl(store_rows_paged_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)rows, ld, (float*)pages, tok_pos,
                       tok_seq, block_table, pages_per_seq, n_tokens, R);
    else if (dtype == PLM_BF16)
        e = launch_pdl(store_rows_paged_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)rows, ld, (bf16*)pages, tok_pos,
                       tok_seq, block_table, pages_per_seq, n_tokens, R);
    else
        return PLM_ERR_DTYPE;
    return plm_status_of(e);
}
