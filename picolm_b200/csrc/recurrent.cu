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

// What a launch of the scan kernel does with the tokens of its segment:
//   SCAN_WHOLE  one segment per sequence: from the cache's state, writes y and the state (decode steps, short prompts)
//   SCAN_LOCAL  from zero, no y: leaves the segment's own contribution to the state and the product of its decays
//   SCAN_FINAL  from the state at the segment's start (put together by scan_combine_kernel), writes y; the last
//               segment of a sequence writes the cache's state
#define SCAN_WHOLE 0
#define SCAN_LOCAL 1
#define SCAN_FINAL 2

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
    int seg_len, max_segs;                // tokens per segment; segments of the longest sequence
    float *seg_state, *seg_decay;         // [seq][segment][H][N][P] and [seq][segment][H][N]
};

// One block per (sequence, head, tile of 32 value columns, segment).  A warp holds 8 columns, two groups of 4; the
// N rows of a column group's state are dealt to 16 lanes (NS consecutive rows each), so a thread keeps NS x 4
// values of the state in registers.  The tokens are taken in order, TC at a time: the block first brings their q,
// k, decay and v to shared memory as fp32 (the exponentials are taken there, once per token and channel), then every
// thread steps its piece of the state through them; y's sum over the rows goes through the 16 lanes by shuffles.
template <typename T, int NS, int MODE, int PASS>
__global__ void __launch_bounds__(SCAN_THREADS) linear_scan_kernel(const ScanArgs a, int TC) {
    constexpr int ROW = NS == 4 ? 4 : NS + 4;             // padded so that a quarter warp's float4 reads hit different banks
    constexpr bool PER_CHANNEL = MODE == DECAY_SIGMOID;
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    int bid = blockIdx.x;
    const int ptile = bid % ptiles;
    bid /= ptiles;
    const int h = bid % a.H, b = bid / a.H;
    const int seg = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int npart = lane & 15, pg = lane >> 4;
    const int pl = (warp << 3) + (pg << 2);               // first of this thread's 4 columns within the tile
    const int p = ptile * SCAN_PTILE + pl;
    const int g = h / a.heads_per_group;
    const int N = a.N, P = a.P;
    float* qs = smem;                                     // [TC][16][ROW]
    float* ks = qs + (long)TC * 16 * ROW;
    float* ds = ks + (long)TC * 16 * ROW;                 // per channel: [TC][16][ROW]; per head: [TC] decay, [TC] scale of v
    float* vs = ds + (PER_CHANNEL ? (long)TC * 16 * ROW : (long)((2 * TC + 3) & ~3));    // [TC][SCAN_PTILE]
    const T* q = (const T*)a.q;
    const T* k = (const T*)a.k;
    const T* v = (const T*)a.v;
    const T* raw = (const T*)a.raw;
    pdl_wait();
    const int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    const int n_segs = PASS == SCAN_WHOLE ? 1 : (s1 - s0 + a.seg_len - 1) / a.seg_len;
    if (PASS == SCAN_LOCAL && seg >= n_segs - 1) return;  // nobody needs what the last segment adds by itself
    if (PASS == SCAN_FINAL && seg >= n_segs) return;
    const int t0 = PASS == SCAN_WHOLE ? s0 : s0 + seg * a.seg_len;
    const int t1 = PASS == SCAN_WHOLE ? s1 : min(s1, t0 + a.seg_len);
    float* st = a.state + (long)a.seq_slot[b] * a.state_stride + (long)h * N * P;
    float* sg = PASS == SCAN_WHOLE ? nullptr : a.seg_state + (((long)b * a.max_segs + seg) * a.H + h) * N * P;
    const float* init = PASS == SCAN_WHOLE ? st : PASS == SCAN_FINAL ? sg : nullptr;
    float S[NS][4];
    float dprod[PER_CHANNEL ? NS : 1];
#pragma unroll
    for (int i = 0; i < (PER_CHANNEL ? NS : 1); ++i) dprod[i] = 1.f;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int n = npart * NS + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) S[i][j] = (init && n < N && p + j < P) ? init[(long)n * P + p + j] : 0.f;
    }
    const float skip = a.skip ? a.skip[h] : 0.f;
    for (int base = t0; base < t1; base += TC) {
        const int nt = min(TC, t1 - base);
        __syncthreads();
#pragma unroll 2
        for (int idx = threadIdx.x; idx < nt * 16 * NS; idx += SCAN_THREADS) {
            const int tt = idx / (16 * NS), n = idx % (16 * NS);
            const int at = (tt * 16 + n / NS) * ROW + n % NS;
            const long row = base + tt;
            const bool in = n < N;
            if (PASS != SCAN_LOCAL) qs[at] = in ? to_f32<T>(q[row * a.ldq + (long)g * N + n]) * a.q_scale : 0.f;
            ks[at] = in ? to_f32<T>(k[row * a.ldk + (long)g * N + n]) : 0.f;
            if (PER_CHANNEL)
                ds[at] = in ? expf(log_sigmoid_f(to_f32<T>(raw[row * a.ldraw + (long)h * N + n]) + a.p0[(long)h * N + n]) * a.power) : 1.f;
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
            const float4 x = *(const float4*)(vs + tt * SCAN_PTILE + pl);
            const float vsc = PER_CHANNEL ? 1.f : ds[TC + tt];
            const float4 vv = make_float4(vsc * x.x, vsc * x.y, vsc * x.z, vsc * x.w);
            const float dh = PER_CHANNEL ? 0.f : ds[tt];
            if (!PER_CHANNEL) dprod[0] *= dh;
            const float4* q4 = (const float4*)(qs + (tt * 16 + npart) * ROW);
            const float4* k4 = (const float4*)(ks + (tt * 16 + npart) * ROW);
            const float4* d4 = (const float4*)(ds + (tt * 16 + npart) * ROW);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i4 = 0; i4 < NS / 4; ++i4) {
                const float4 kk = k4[i4];
                float4 qq = make_float4(0.f, 0.f, 0.f, 0.f), dd = make_float4(dh, dh, dh, dh);
                if (PASS != SCAN_LOCAL) qq = q4[i4];
                if (PER_CHANNEL) dd = d4[i4];
                const float kr[4] = {kk.x, kk.y, kk.z, kk.w}, qr[4] = {qq.x, qq.y, qq.z, qq.w}, dr[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float* Sr = S[4 * i4 + r];
                    if (PER_CHANNEL) dprod[4 * i4 + r] *= dr[r];
                    Sr[0] = fmaf(dr[r], Sr[0], kr[r] * vv.x);
                    Sr[1] = fmaf(dr[r], Sr[1], kr[r] * vv.y);
                    Sr[2] = fmaf(dr[r], Sr[2], kr[r] * vv.z);
                    Sr[3] = fmaf(dr[r], Sr[3], kr[r] * vv.w);
                    if (PASS != SCAN_LOCAL) {
                        acc.x = fmaf(Sr[0], qr[r], acc.x);
                        acc.y = fmaf(Sr[1], qr[r], acc.y);
                        acc.z = fmaf(Sr[2], qr[r], acc.z);
                        acc.w = fmaf(Sr[3], qr[r], acc.w);
                    }
                }
            }
            if (PASS != SCAN_LOCAL) {
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) {
                    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
                    acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
                    acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
                    acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
                }
                if (npart == 0) {
                    float* yr = a.y + (long)(base + tt) * a.ldy + (long)h * P + p;
                    const float out[4] = {fmaf(skip, x.x, acc.x), fmaf(skip, x.y, acc.y), fmaf(skip, x.z, acc.z), fmaf(skip, x.w, acc.w)};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (p + j < P) yr[j] = out[j];
                }
            }
        }
    }
    float* dst = PASS == SCAN_LOCAL ? sg : (PASS == SCAN_WHOLE || seg == n_segs - 1) ? st : nullptr;
    if (dst) {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int n = npart * NS + i;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (n < N && p + j < P) dst[(long)n * P + p + j] = S[i][j];
        }
    }
    if (PASS == SCAN_LOCAL && ptile == 0 && warp == 0 && pg == 0) {
        float* dd = a.seg_decay + (((long)b * a.max_segs + seg) * a.H + h) * N;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            const int n = npart * NS + i;
            if (n < N) dd[n] = PER_CHANNEL ? dprod[PER_CHANNEL ? i : 0] : dprod[0];
        }
    }
}

// Between the two passes over the segments: the state at the start of every segment, from the cache's state and
// what the segments before it add: S_in[0] = state, S_in[c + 1] = decay[c] * S_in[c] + local[c].  One thread per
// element of a sequence's state; S_in[c] takes local[c]'s place.
__global__ void scan_combine_kernel(const ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const long per_seq = (long)a.H * a.N * a.P;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per_seq * a.n_seqs) return;
    const int b = (int)(idx / per_seq);
    const long e = idx % per_seq;
    const long hn = e / a.P;
    const int n_segs = (a.seq_start[b + 1] - a.seq_start[b] + a.seg_len - 1) / a.seg_len;
    float S = a.state[(long)a.seq_slot[b] * a.state_stride + e];
    float* sg = a.seg_state + (long)b * a.max_segs * per_seq + e;
    const float* dd = a.seg_decay + (long)b * a.max_segs * a.H * a.N + hn;
    for (int c = 0; c < n_segs; ++c) {
        const float local = c < n_segs - 1 ? sg[(long)c * per_seq] : 0.f;
        sg[(long)c * per_seq] = S;
        if (c < n_segs - 1) S = fmaf(dd[(long)c * a.H * a.N], S, local);
    }
}

template <int NS>
static size_t scan_smem(int mode, int* TC) {
    const int ROW = NS == 4 ? 4 : NS + 4;
    // tokens per pass: as many as fit into about 40 KB of shared memory, 16 at most
    const long per_token = (mode == DECAY_SIGMOID ? 3L : 2L) * 16 * ROW + SCAN_PTILE + (mode == DECAY_SIGMOID ? 0 : 2);
    int tc = (int)((40 * 1024 / 4 - 4) / per_token);
    tc = tc > 16 ? 16 : tc < 1 ? 1 : tc;
    *TC = tc;
    return (size_t)(per_token * tc + 4) * sizeof(float);
}

template <typename T, int NS, int MODE>
static cudaError_t scan_launch(const ScanArgs& a, cudaStream_t stream) {
    int TC;
    const size_t smem = scan_smem<NS>(MODE, &TC);
    const int ptiles = (a.P + SCAN_PTILE - 1) / SCAN_PTILE;
    const unsigned blocks = (unsigned)((long)a.n_seqs * a.H * ptiles);
    if (a.max_segs <= 1)
        return launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_WHOLE>, dim3(blocks), dim3(SCAN_THREADS), smem, stream, a, TC);
    cudaError_t e = launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_LOCAL>, dim3(blocks, a.max_segs - 1), dim3(SCAN_THREADS), smem,
                               stream, a, TC);
    if (e != cudaSuccess) return e;
    const long elems = (long)a.n_seqs * a.H * a.N * a.P;
    e = launch_pdl(scan_combine_kernel, dim3((unsigned)((elems + 255) / 256)), dim3(256), 0, stream, a);
    if (e != cudaSuccess) return e;
    return launch_pdl(linear_scan_kernel<T, NS, MODE, SCAN_FINAL>, dim3(blocks, a.max_segs), dim3(SCAN_THREADS), smem, stream, a, TC);
}

template <typename T>
static int scan_dispatch(const ScanArgs& a, int mode, cudaStream_t stream) {
    const int ns = (a.N + 15) / 16;
    cudaError_t e;
#define SCAN_NS(NS_) (mode == DECAY_SIGMOID ? scan_launch<T, NS_, DECAY_SIGMOID>(a, stream) : scan_launch<T, NS_, DECAY_STEP>(a, stream))
    if (ns <= 4) e = SCAN_NS(4);
    else if (ns <= 8) e = SCAN_NS(8);
    else if (ns <= 16) e = SCAN_NS(16);
    else return PLM_ERR_UNSUPPORTED;
#undef SCAN_NS
    return plm_status_of(e);
}

// How a step whose longest sequence brings `max_new` tokens is cut: out[0] tokens per segment, out[1] segments of the
// longest sequence (1: one pass from the cache's state, no scratch memory).  Segments are worth their second pass
// when the sequences alone leave most of the GPU idle; there are as many as give every SM a few blocks, each of at
// least 64 tokens, and no more than keep the scratch memory under 1 GiB.
extern "C" int plm_linear_scan_plan(int n_seqs, int H, int N, int P, int max_new, int* out) {
    out[0] = max_new > 0 ? max_new : 1;
    out[1] = 1;
    if (n_seqs <= 0 || H <= 0 || N <= 0 || P <= 0) return PLM_ERR_SHAPE;
    if (max_new < 192) return PLM_OK;
    const long blocks = (long)n_seqs * H * ((P + SCAN_PTILE - 1) / SCAN_PTILE);
    long segs = (6L * PLM_SM_COUNT + blocks - 1) / blocks;
    const long most = max_new / 64;
    if (segs > most) segs = most;
    const long state_bytes = (long)n_seqs * H * N * (P + 1) * 4;
    while (segs > 1 && segs * state_bytes > (1L << 30)) --segs;
    if (segs <= 1) return PLM_OK;
    int len = (int)((max_new + segs - 1) / segs);
    len = (len + 15) / 16 * 16;
    out[0] = len;
    out[1] = (max_new + len - 1) / len;
    return PLM_OK;
}

extern "C" int plm_linear_scan(const void* q, const void* k, const void* v, const void* raw, int dtype, long ldq, long ldk,
                               long ldv, long ldraw, int mode, const float* p0, const float* p1, const float* skip,
                               float q_scale, float power, float* state, long state_stride, float* y, long ldy,
                               const int* seq_start, const int* seq_slot, int n_seqs, int H, int N, int P,
                               int heads_per_group, int seg_len, int max_segs, float* seg_state, float* seg_decay,
                               cudaStream_t stream) {
    if (n_seqs <= 0 || H <= 0 || N <= 0 || P <= 0 || heads_per_group <= 0) return PLM_ERR_SHAPE;
    if (mode != DECAY_STEP && mode != DECAY_SIGMOID) return PLM_ERR_UNSUPPORTED;
    if (mode == DECAY_STEP && !p1) return PLM_ERR_SHAPE;
    if (!p0) return PLM_ERR_SHAPE;
    if (N > 256) return PLM_ERR_UNSUPPORTED;
    if (max_segs > 1 && (!seg_state || !seg_decay || seg_len <= 0 || max_segs > 65535)) return PLM_ERR_SHAPE;
    ScanArgs a;
    a.q = q, a.k = k, a.v = v, a.raw = raw;
    a.ldq = ldq, a.ldk = ldk, a.ldv = ldv, a.ldraw = ldraw;
    a.p0 = p0, a.p1 = p1, a.skip = skip;
    a.q_scale = q_scale, a.power = power;
    a.state = state, a.state_stride = state_stride;
    a.y = y, a.ldy = ldy;
    a.seq_start = seq_start, a.seq_slot = seq_slot;
    a.n_seqs = n_seqs, a.H = H, a.N = N, a.P = P, a.heads_per_group = heads_per_group;
    a.seg_len = seg_len, a.max_segs = max_segs < 1 ? 1 : max_segs;
    a.seg_state = seg_state, a.seg_decay = seg_decay;
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
#pragma unroll 4
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
#pragma unroll 4
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
