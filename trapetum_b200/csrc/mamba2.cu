// A selective state-space mixer (the Mamba-2 recurrence) between its input and output products.
//
// The input product gives a row [z: inner | xBC: channels] per token in the compute dtype and the step sizes
// [dt: heads] in 32-bit (they enter an exponential), inner = heads * P, channels = inner + 2 * groups * N.
// Three kernels:
//
//   tb_mamba2_conv       u = silu(bias + sum_j w[c][j] * in[t - (taps-1) + j][c]) over the token's own sequence,
//                        rows before the step's first token come from the sequence's state (zeros at its start);
//                        then the state takes the last taps-1 inputs.  One token per sequence: one launch does both.
//   tb_mamba2_scan       per head h (group g = h / (heads / groups)), with dt = softplus(dt_raw + dt_bias):
//                          S <- exp(-exp(A_log[h]) dt) S + dt * x_t B_t^T      S is [P][N]
//                          y_t = S C_t + D[h] x_t
//                        sequential over a sequence's tokens, S read from and written back to the state.  Where few
//                        long prompts would leave most SMs idle, a prompt is cut into chunks: one launch runs the
//                        recurrence of every chunk but the last from zero and keeps its end state and the product of
//                        its decays, a second launch starts every chunk from what the chunks before it left
//                        (S_c = D_(c-1) S_(c-1) + E_(c-1), folded by the chunk itself) and writes y.  Twice the
//                        arithmetic, chunks times the parallelism; the same sums in another order.
//   tb_mamba2_gate_norm  out = groupnorm(y * silu(z)) * w, the norm over `norm_groups` equal parts of a row.
//
// The state of a sequence is one 32-bit row: [heads][P][N] of S, then [taps-1][channels] of conv inputs
// (oldest first).  The convolution and its silu work on the compute dtype's values with 32-bit sums; softplus,
// the decay, S, y and the gated norm are 32-bit throughout.
#include "common.cuh"

TB_EXPORT_ERROR()

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

struct Mamba2Args {
    const void* proj; long long proj_stride;      // [tokens][inner + channels], compute dtype
    const float* dt; long long dt_stride;          // [tokens][heads], the step sizes before bias and softplus,
    int dt_splits; long long dt_split_stride;      // as dt_splits partial sums (added in split order)
    int heads, P, N, groups, taps, norm_groups;
    const void* conv_w; const void* conv_b;        // [channels][taps], [channels]   (weights' dtype)
    const void* dt_bias; const void* A_log; const void* D;   // [heads]
    const void* norm_w;                            // [inner]
    float eps;
    float* state; long long state_stride;          // [slots][state_stride]
    const int* seq_start; const int* token_seq; const int* slot_ids;
    void* xbc;                                     // [tokens][channels], compute dtype (conv output)
    float* y;                                      // [tokens][inner]
    void* out;                                     // [tokens][inner], compute dtype
    int batch, n_tokens;
    // a long prompt cut into chunks that run side by side (see mamba2_scan_kernel): end states [batch][n_chunks][heads*P*N],
    // decay products [batch][n_chunks][heads], tokens per chunk (a multiple of the tile), chunks per sequence
    float* chunk_state; float* chunk_decay; int chunk_len; int n_chunks;
};

// ---------------------------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void mamba2_conv_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int inner = a.heads * a.P, ch = inner + 2 * a.groups * a.N;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= ch) return;
    const int b = a.token_seq[t];
    const int i = t - a.seq_start[b];                               // the token's index among the step's tokens of its sequence
    const float* st = a.state + (size_t)a.slot_ids[b] * a.state_stride + (size_t)a.heads * a.P * a.N;
    const T* in = (const T*)a.proj + inner + c;
    const TW* w = (const TW*)a.conv_w + (size_t)c * a.taps;
    float acc = to_f<TW>(((const TW*)a.conv_b)[c]);
    for (int j = 0; j < a.taps; j++) {
        const int d = i - (a.taps - 1) + j;                          // index among the step's tokens; negative: from the state
        const float v = d >= 0 ? to_f<T>(in[(size_t)(t - (a.taps - 1) + j) * a.proj_stride])
                               : st[(size_t)(a.taps - 1 + d) * ch + c];
        acc += to_f<TW>(w[j]) * v;
    }
    ((T*)a.xbc)[(size_t)t * ch + c] = from_f<T>(silu_f(acc));
}

// After a step of several tokens: the state keeps the last taps-1 inputs of each sequence.  One thread owns a
// (sequence, channel) column and shifts it in ascending order, so the update is safe in place.
template <typename T>
__global__ void mamba2_conv_state_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int inner = a.heads * a.P, ch = inner + 2 * a.groups * a.N;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int b = blockIdx.x;
    if (c >= ch) return;
    const int s0 = a.seq_start[b], n = a.seq_start[b + 1] - s0, keep = a.taps - 1;
    float* st = a.state + (size_t)a.slot_ids[b] * a.state_stride + (size_t)a.heads * a.P * a.N;
    const T* in = (const T*)a.proj + inner + c;
    for (int j = 0; j < keep; j++) {
        const int d = n - keep + j;                                  // index among the step's tokens
        st[(size_t)j * ch + c] = d >= 0 ? to_f<T>(in[(size_t)(s0 + d) * a.proj_stride]) : st[(size_t)(j + n) * ch + c];
    }
}

// One token per sequence: convolution and state shift by the thread that owns the column.
template <typename T, typename TW>
__global__ void mamba2_conv_step_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int inner = a.heads * a.P, ch = inner + 2 * a.groups * a.N;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int b = blockIdx.x;                                        // token b belongs to sequence b
    if (c >= ch) return;
    const int keep = a.taps - 1;
    float* st = a.state + (size_t)a.slot_ids[b] * a.state_stride + (size_t)a.heads * a.P * a.N;
    const TW* w = (const TW*)a.conv_w + (size_t)c * a.taps;
    const float cur = to_f<T>(((const T*)a.proj)[(size_t)b * a.proj_stride + inner + c]);
    float acc = to_f<TW>(((const TW*)a.conv_b)[c]);
    for (int j = 0; j < keep; j++) {
        const float v = st[(size_t)j * ch + c];
        acc += to_f<TW>(w[j]) * v;
        if (j > 0) st[(size_t)(j - 1) * ch + c] = v;
    }
    acc += to_f<TW>(w[keep]) * cur;
    if (keep > 0) st[(size_t)(keep - 1) * ch + c] = cur;
    ((T*)a.xbc)[(size_t)b * ch + c] = from_f<T>(silu_f(acc));
}

// ---------------------------------------------------------------------------------------------------------
// The recurrence.  A CTA owns (sequence, head, PT values of P): thread (pl, ns) keeps the states S[p][n] of two
// neighbouring p with n = (k * 8 + ns) * 4 + e (k < NV, e < 4) in registers, so that the eight threads of a pair read
// B and C of a token as eight neighbouring 16-byte words of shared memory (no bank conflict) and use each word for
// both p.  B, C,
// x, dt and the decay of TT tokens at a time are staged in shared memory; the next tile's values are requested into
// registers before this tile's steps run, so that the loads' latency hides behind the recurrence.  A thread's parts of
// the 2 TT outputs stay in registers and are added over the eight threads once per tile, off the dependency chain, by
// a butterfly in which every thread hands over half of what it holds at each of the three stages.
#define SCAN_NS 8
#define SCAN_TT 16
#define SCAN_PP 2

template <typename T> struct Chunk8;                                 // eight neighbouring values of the compute dtype
template <> struct Chunk8<bf16> {
    uint4 v;
    __device__ __forceinline__ void load(const bf16* p) { v = *(const uint4*)p; }
    __device__ __forceinline__ void zero() { v = make_uint4(0, 0, 0, 0); }
    __device__ __forceinline__ void store(float* d) const {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
        *(float4*)d = make_float4(f[0], f[1], f[2], f[3]);
        *(float4*)(d + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};
template <> struct Chunk8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *(const float4*)p; b = *(const float4*)(p + 4); }
    __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void store(float* d) const { *(float4*)d = a; *(float4*)(d + 4) = b; }
};

// VEC8: N is a multiple of 8 and the rows of B and C start on 16-byte boundaries.
// MODE 0: a whole sequence per CTA.  MODE 1: a chunk from zero (the first chunk: from the sequence's state, of which it
// also leaves a copy in the last chunk's slot, which is otherwise unused), end state and decay product kept, no y;
// the last chunk of a sequence does nothing.  MODE 2: a chunk from the folded states of the chunks before it, y
// written; the last chunk writes the sequence's state (only it reads it in this launch: a sequence of one chunk).
template <typename T, typename TW, int NV, int PT, bool VEC8, int MODE>
__global__ void __launch_bounds__(SCAN_NS * PT / SCAN_PP) mamba2_scan_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    constexpr int NP = NV * 32;                                      // padded state size (zeros beyond N)
    constexpr int THREADS = SCAN_NS * PT / SCAN_PP;
    constexpr int CHUNKS = SCAN_TT * 2 * NP / 8;                     // 8-value chunks of B and C in a tile
    constexpr int CPT = (CHUNKS + THREADS - 1) / THREADS;            // chunks a thread fetches
    constexpr int XPT = SCAN_TT * PT / THREADS;                      // x values a thread fetches (4)
    extern __shared__ __align__(16) float sh[];                      // [TT][NP] B, [TT][NP] C, [TT][PT] x, [TT][2] dt and decay
    const int N = a.N, P = a.P, H = a.heads;
    const int inner = H * P, ch = inner + 2 * a.groups * N;
    const int b = MODE == 0 ? blockIdx.z : blockIdx.z / a.n_chunks, chunk = MODE == 0 ? 0 : blockIdx.z % a.n_chunks;
    const int h = blockIdx.y, p0 = blockIdx.x * PT;
    const int g = h / (H / a.groups);
    const int ns = threadIdx.x % SCAN_NS, pl = threadIdx.x / SCAN_NS;
    const int p = p0 + pl * SCAN_PP;                                 // this thread's first p
    float* sB = sh;
    float* sC = sh + SCAN_TT * NP;
    float* sx = sC + SCAN_TT * NP;
    float* sdt = sx + SCAN_TT * PT;
    const float A = -expf(to_f<TW>(((const TW*)a.A_log)[h]));
    const float Dh = to_f<TW>(((const TW*)a.D)[h]);
    const float dtb = to_f<TW>(((const TW*)a.dt_bias)[h]);
    pdl_wait();
    int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    bool last = true;
    if (MODE != 0) {                                                 // this CTA's chunk of the sequence
        const int end = s1;
        s0 += chunk * a.chunk_len;
        if (s0 >= end) return;                                       // (the same in every thread)
        s1 = min(end, s0 + a.chunk_len);
        last = s1 == end;
        if (MODE == 1 && last) return;
    }
    float* S = a.state + (size_t)a.slot_ids[b] * a.state_stride + (size_t)h * P * N;
    const size_t hpn = (size_t)H * P * N;
    float* E = MODE == 0 ? nullptr : a.chunk_state + (size_t)b * a.n_chunks * hpn + (size_t)h * P * N;   // chunk 0's slot, this head
    float s[SCAN_PP][NV][4];
    auto each = [&](auto&& f) {                                      // f(j, k, e, offset in [P][N]) for the states this thread owns
#pragma unroll
        for (int j = 0; j < SCAN_PP; j++)
#pragma unroll
            for (int k = 0; k < NV; k++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int n = (k * SCAN_NS + ns) * 4 + e;
                    if (p + j < P && n < N) f(j, k, e, (size_t)(p + j) * N + n);
                }
    };
#pragma unroll
    for (int j = 0; j < SCAN_PP; j++)
#pragma unroll
        for (int k = 0; k < NV; k++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][k][e] = 0.f;
    if (MODE == 0 || (MODE == 2 && chunk == 0 && last)) {
        each([&](int j, int k, int e, size_t o) { s[j][k][e] = S[o]; });
    } else if (MODE == 1) {
        if (chunk == 0) each([&](int j, int k, int e, size_t o) { s[j][k][e] = S[o]; E[(size_t)(a.n_chunks - 1) * hpn + o] = S[o]; });
    } else if (chunk == 0) {
        each([&](int j, int k, int e, size_t o) { s[j][k][e] = E[(size_t)(a.n_chunks - 1) * hpn + o]; });
    } else {
        for (int c = 0; c < chunk; c++) {                            // the first chunk's end state holds the sequence's state already
            const float d = c == 0 ? 0.f : a.chunk_decay[((size_t)b * a.n_chunks + c) * H + h];
            const float* Ec = E + (size_t)c * hpn;
            each([&](int j, int k, int e, size_t o) { s[j][k][e] = d * s[j][k][e] + Ec[o]; });
        }
    }
    float decay = 1.f;
    const T* xbc = (const T*)a.xbc;

    Chunk8<T> pre[VEC8 ? CPT : 1];
    float pre_x[XPT], pre_dt = 0.f;
    auto fetch = [&](int tb) {                                       // the tile that starts at token tb, into registers
        const int nt = min(SCAN_TT, s1 - tb);
        if (VEC8) {
#pragma unroll
            for (int l = 0; l < CPT; l++) {
                const int c = threadIdx.x + l * THREADS;
                const int tt = c / (2 * NP / 8), r = c % (2 * NP / 8);
                const int n8 = (r % (NP / 8)) * 8;
                pre[l].zero();
                if (c < CHUNKS && tt < nt && n8 < N)
                    pre[l].load(xbc + (size_t)(tb + tt) * ch + inner + g * N + (r >= NP / 8 ? a.groups * N : 0) + n8);
            }
        }
#pragma unroll
        for (int l = 0; l < XPT; l++) {
            const int i = threadIdx.x + l * THREADS;
            const int tt = i / PT, pp = p0 + i % PT;
            pre_x[l] = (tt < nt && pp < P) ? to_f<T>(xbc[(size_t)(tb + tt) * ch + h * P + pp]) : 0.f;
        }
        if (threadIdx.x < nt) {
            const float* q = a.dt + (size_t)(tb + threadIdx.x) * a.dt_stride + h;
            pre_dt = q[0];
            for (int sp = 1; sp < a.dt_splits; sp++) pre_dt += q[(size_t)sp * a.dt_split_stride];
        }
    };
    auto commit = [&](int tb) {                                      // registers (or, without VEC8, memory) to shared memory
        const int nt = min(SCAN_TT, s1 - tb);
        if (VEC8) {
#pragma unroll
            for (int l = 0; l < CPT; l++) {
                const int c = threadIdx.x + l * THREADS;
                const int tt = c / (2 * NP / 8), r = c % (2 * NP / 8);
                if (c < CHUNKS) pre[l].store((r >= NP / 8 ? sC : sB) + tt * NP + (r % (NP / 8)) * 8);
            }
        } else {
            for (int i = threadIdx.x; i < nt * NP; i += THREADS) {
                const int tt = i / NP, n = i % NP;
                const T* row = xbc + (size_t)(tb + tt) * ch + inner + g * N;
                sB[i] = n < N ? to_f<T>(row[n]) : 0.f;
                sC[i] = n < N ? to_f<T>(row[a.groups * N + n]) : 0.f;
            }
        }
#pragma unroll
        for (int l = 0; l < XPT; l++) sx[threadIdx.x + l * THREADS] = pre_x[l];
        if (threadIdx.x < nt) {
            const float dt = softplus_f(pre_dt + dtb);
            sdt[2 * threadIdx.x] = dt;
            sdt[2 * threadIdx.x + 1] = expf(A * dt);
        }
    };

    if (s0 < s1) fetch(s0);
    for (int tb = s0; tb < s1; tb += SCAN_TT) {
        const int nt = min(SCAN_TT, s1 - tb);
        __syncthreads();                                             // the last tile's steps have read shared memory
        commit(tb);
        __syncthreads();
        if (tb + SCAN_TT < s1) fetch(tb + SCAN_TT);
        float yp[SCAN_TT * SCAN_PP];                                 // yp[tt * 2 + j]: this thread's part of y of token tt, p + j
#pragma unroll
        for (int tt = 0; tt < SCAN_TT; tt++) {
            yp[2 * tt] = yp[2 * tt + 1] = 0.f;
            if (tt < nt) {                                           // the same in every thread of the CTA
                const float dec = sdt[2 * tt + 1], dt = sdt[2 * tt];
                if (MODE == 1) decay *= dec;
                const float dx0 = dt * sx[tt * PT + pl * SCAN_PP], dx1 = dt * sx[tt * PT + pl * SCAN_PP + 1];
                const float4* Bt = (const float4*)(sB + tt * NP);
                const float4* Ct = (const float4*)(sC + tt * NP);
                float y0[4] = {0.f, 0.f, 0.f, 0.f}, y1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < NV; k++) {
                    const float4 bv = Bt[k * SCAN_NS + ns], cv = Ct[k * SCAN_NS + ns];
                    const float bb[4] = {bv.x, bv.y, bv.z, bv.w}, cc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        s[0][k][e] = dec * s[0][k][e] + dx0 * bb[e]; y0[e] += s[0][k][e] * cc[e];
                        s[1][k][e] = dec * s[1][k][e] + dx1 * bb[e]; y1[e] += s[1][k][e] * cc[e];
                    }
                }
                yp[2 * tt] = (y0[0] + y0[1]) + (y0[2] + y0[3]);
                yp[2 * tt + 1] = (y1[0] + y1[1]) + (y1[2] + y1[3]);
            }
        }
        if (MODE != 1) {                                             // (end states only: no outputs)
        // the eight threads of a pair add their parts: at each stage a thread keeps one half of its values and hands
        // the other to its partner; thread ns ends with the sums of tokens 2 ns and 2 ns + 1, both p
#pragma unroll
        for (int o = SCAN_NS / 2, half = SCAN_TT * SCAN_PP / 2; o > 0; o >>= 1, half >>= 1) {
            const bool up = (ns & o) != 0;
#pragma unroll
            for (int i = 0; i < SCAN_TT * SCAN_PP / 2; i++) {
                if (i < half) {
                    const float keep = up ? yp[i + half] : yp[i];
                    const float send = up ? yp[i] : yp[i + half];
                    yp[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int tt = 2 * ns + (r >> 1), j = r & 1;
            if (tt < nt && p + j < P)
                a.y[(size_t)(tb + tt) * inner + h * P + p + j] = yp[r] + Dh * sx[tt * PT + pl * SCAN_PP + j];
        }
        }
    }
    if (MODE == 1) {
        each([&](int j, int k, int e, size_t o) { E[(size_t)chunk * hpn + o] = s[j][k][e]; });
        if (blockIdx.x == 0 && threadIdx.x == 0) a.chunk_decay[((size_t)b * a.n_chunks + chunk) * H + h] = decay;
    } else if (last) {
        each([&](int j, int k, int e, size_t o) { S[o] = s[j][k][e]; });
    }
}

// ---------------------------------------------------------------------------------------------------------
// out = groupnorm(y * silu(z)) * w: one CTA per (token, norm group).
template <typename T, typename TW>
__global__ void mamba2_gate_norm_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int inner = a.heads * a.P, gs = inner / a.norm_groups;
    const int t = blockIdx.x, c0 = blockIdx.y * gs;
    const float* y = a.y + (size_t)t * inner + c0;
    const T* z = (const T*)a.proj + (size_t)t * a.proj_stride + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = y[i] * silu_f(to_f<T>(z[i]));
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)gs + a.eps);
    const TW* w = (const TW*)a.norm_w + c0;
    T* out = (T*)a.out + (size_t)t * inner + c0;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = y[i] * silu_f(to_f<T>(z[i]));
        out[i] = from_f<T>(v * r * to_f<TW>(w[i]));
    }
}

// The same for few tokens, where the launch's time is its chain of memory round trips: a thread keeps its NV groups
// of four columns in registers, so y and z are read once (group sizes up to 1,024 x 4 x NV that are multiples of 4).
template <typename T, typename TW, int NV>
__global__ void __launch_bounds__(1024) mamba2_gate_norm_few_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    __shared__ float red[33];
    const int inner = a.heads * a.P, gs = inner / a.norm_groups;
    const int t = blockIdx.x, c0 = blockIdx.y * gs;
    float w[NV][4], v[NV][4];
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) w[k][e] = i < gs ? to_f<TW>(((const TW*)a.norm_w)[c0 + i + e]) : 0.f;
    }
    pdl_wait();
    const float* y = a.y + (size_t)t * inner + c0;
    const T* z = (const T*)a.proj + (size_t)t * a.proj_stride + c0;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) v[k][e] = 0.f;
        if (i < gs) {
            const float4 yy = *(const float4*)(y + i);
            const float ye[4] = {yy.x, yy.y, yy.z, yy.w};
#pragma unroll
            for (int e = 0; e < 4; e++) { v[k][e] = ye[e] * silu_f(to_f<T>(z[i + e])); ss += v[k][e] * v[k][e]; }
        }
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)gs + a.eps);
    T* out = (T*)a.out + (size_t)t * inner + c0;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < gs) {
#pragma unroll
            for (int e = 0; e < 4; e++) out[i + e] = from_f<T>(v[k][e] * r * w[k][e]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
static int check(const Mamba2Args& a) {
    if (a.heads <= 0 || a.P <= 0 || a.N <= 0 || a.groups <= 0 || a.taps <= 0 || a.norm_groups <= 0)
        return tb_refuse("mamba2: heads=%d P=%d N=%d groups=%d taps=%d norm_groups=%d", a.heads, a.P, a.N, a.groups, a.taps,
                         a.norm_groups);
    if (a.heads % a.groups) return tb_refuse("mamba2: %d heads cannot share %d groups", a.heads, a.groups);
    if ((a.heads * a.P) % a.norm_groups) return tb_refuse("mamba2: %d inner columns do not split into %d norm groups",
                                                          a.heads * a.P, a.norm_groups);
    if (a.N > 256) return tb_refuse("mamba2: state size %d (at most 256)", a.N);
    return 0;
}

// The small tensors (taps, biases, A_log, D, the norm's weight) enter 32-bit arithmetic and are taken in 32 bits.
#define DISPATCH2(ct, cw, ...)                                                             \
    do {                                                                                   \
        if ((cw) != TB_F32) return tb_refuse("mamba2: the small tensors must be float32 (code %d)", (cw)); \
        if ((ct) == TB_F32) { typedef float T; typedef float TW; __VA_ARGS__; }            \
        else if ((ct) == TB_BF16) { typedef bf16 T; typedef float TW; __VA_ARGS__; }       \
        else return tb_refuse("mamba2: unknown dtype code %d", (ct));                      \
    } while (0)

extern "C" int tb_mamba2_conv(const Mamba2Args* args, int dtype, int w_dtype, int one_token_each, cudaStream_t stream) {
    Mamba2Args a = *args;
    if (a.n_tokens <= 0) return 0;
    if (check(a)) return -1;
    const int ch = a.heads * a.P + 2 * a.groups * a.N;
    const unsigned gy = (ch + 127) / 128;
    if (one_token_each) {
        DISPATCH2(dtype, w_dtype, tb_launch(mamba2_conv_step_kernel<T, TW>, dim3(a.batch, gy), dim3(128), 0, stream, a));
        return tb_launch_status();
    }
    DISPATCH2(dtype, w_dtype, tb_launch(mamba2_conv_kernel<T, TW>, dim3(a.n_tokens, gy), dim3(128), 0, stream, a));
    int st = tb_launch_status();
    if (st) return st;
    if (a.taps > 1) {
        TB_DISPATCH_1(dtype, T, tb_launch(mamba2_conv_state_kernel<T>, dim3(a.batch, gy), dim3(128), 0, stream, a));
    }
    return tb_launch_status();
}

static int scan_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0; cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

// Into how many chunks (and of how many tokens) the longest prompt of a step is cut: 1 unless the (sequence, head,
// 32 values of P) tiles are fewer than four an SM and the prompt is long enough for chunks of 128 tokens and more.
extern "C" int tb_mamba2_plan(int heads, int P, int batch, int max_seq_len, int* chunk_len) {
    const long long tiles = (long long)((P + 31) / 32) * heads * batch;
    const int sms = scan_sms();
    int chunks = 1;
    if (tiles < 4LL * sms && max_seq_len >= 256) {
        chunks = (int)((6LL * sms + tiles - 1) / tiles);
        if (chunks > max_seq_len / 128) chunks = max_seq_len / 128;
        if (chunks > 64) chunks = 64;
    }
    int len = (max_seq_len + chunks - 1) / chunks;
    len = (len + SCAN_TT - 1) / SCAN_TT * SCAN_TT;
    if (len < SCAN_TT) len = SCAN_TT;
    chunks = (max_seq_len + len - 1) / len;
    if (chunks < 1) chunks = 1;
    if (chunk_len) *chunk_len = len;
    return chunks;
}

extern "C" int tb_mamba2_scan(const Mamba2Args* args, int dtype, int w_dtype, cudaStream_t stream) {
    Mamba2Args a = *args;
    if (a.n_tokens <= 0) return 0;
    if (check(a)) return -1;
    const int sms = scan_sms();
    const bool chunked = a.n_chunks > 1;
    if (chunked && (a.chunk_state == nullptr || a.chunk_decay == nullptr || a.chunk_len < SCAN_TT || a.chunk_len % SCAN_TT))
        return tb_refuse("mamba2: chunks need their scratch and a length that is a multiple of %d", SCAN_TT);
    const int zdim = a.batch * (chunked ? a.n_chunks : 1);
    // thirty-two values of P a CTA (128 threads), or sixteen where that would leave SMs without work
    const int pt = ((long long)((a.P + 31) / 32) * a.heads * zdim >= 2LL * sms) ? 32 : 16;
    const dim3 grid((a.P + pt - 1) / pt, a.heads, zdim);
    if (grid.y > 65535 || grid.z > 65535) return tb_refuse("mamba2: too many heads or sequences for one launch");
    const int nv = (a.N + 31) / 32;
    const int es = dtype == TB_BF16 ? 2 : 4;
    const int chn = a.heads * a.P + 2 * a.groups * a.N;
    const bool vec8 = a.N % 8 == 0 && ((size_t)chn * es) % 16 == 0 && ((size_t)a.heads * a.P * es) % 16 == 0 &&
                      ((uintptr_t)a.xbc & 15) == 0;
#define SCAN4(NV_, PT_, V8_, MODE_) \
        DISPATCH2(dtype, w_dtype, tb_launch(mamba2_scan_kernel<T, TW, NV_, PT_, V8_, MODE_>, dim3(grid), dim3(SCAN_NS * (PT_) / SCAN_PP), smem, stream, a))
#define SCAN3(NV_, PT_, MODE_) do { \
        const size_t smem = (size_t)(SCAN_TT * 2 * (NV_) * 32 + SCAN_TT * (PT_) + SCAN_TT * 2) * sizeof(float); \
        if (vec8) SCAN4(NV_, PT_, true, MODE_); else SCAN4(NV_, PT_, false, MODE_); \
    } while (0)
#define SCAN2(NV_, MODE_) do { if (pt == 32) SCAN3(NV_, 32, MODE_); else SCAN3(NV_, 16, MODE_); } while (0)
#define SCAN(MODE_) do { if (nv <= 1) SCAN2(1, MODE_); else if (nv <= 2) SCAN2(2, MODE_); else if (nv <= 4) SCAN2(4, MODE_); else SCAN2(8, MODE_); } while (0)
    if (!chunked) {
        SCAN(0);
        return tb_launch_status();
    }
    SCAN(1);
    const int st = tb_launch_status();
    if (st) return st;
    SCAN(2);
#undef SCAN
#undef SCAN2
#undef SCAN3
#undef SCAN4
    return tb_launch_status();
}

extern "C" int tb_mamba2_gate_norm(const Mamba2Args* args, int dtype, int w_dtype, cudaStream_t stream) {
    Mamba2Args a = *args;
    if (a.n_tokens <= 0) return 0;
    if (check(a)) return -1;
    const int gs = a.heads * a.P / a.norm_groups;
    int threads = (gs + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
    if (a.norm_groups > 65535) return tb_refuse("mamba2: too many norm groups");
    if (a.n_tokens <= 64 && gs % 4 == 0 && gs <= 1024 * 4 * 4 && (a.heads * a.P) % 4 == 0 && ((uintptr_t)a.y & 15) == 0) {
        const int groups4 = gs / 4;
        const int nvv = groups4 <= 1024 ? 1 : groups4 <= 2048 ? 2 : 4;
        int th = ((groups4 + nvv - 1) / nvv + 31) / 32 * 32;
        if (th < 64) th = 64;
#define FEW(NV_) DISPATCH2(dtype, w_dtype, tb_launch(mamba2_gate_norm_few_kernel<T, TW, NV_>, dim3(a.n_tokens, a.norm_groups), dim3(th), 0, stream, a))
        if (nvv == 1) FEW(1); else if (nvv == 2) FEW(2); else FEW(4);
#undef FEW
        return tb_launch_status();
    }
    DISPATCH2(dtype, w_dtype, tb_launch(mamba2_gate_norm_kernel<T, TW>, dim3(a.n_tokens, a.norm_groups), dim3(threads), 0, stream, a));
    return tb_launch_status();
}
