// A selective state-space mixer (the Mamba-2 recurrence) between its input and output products.
//
// The input product gives a row [z: inner | xBC: channels | dt: heads] per token, inner = heads * P,
// channels = inner + 2 * groups * N.  Three kernels:
//
//   tb_mamba2_conv       u = silu(bias + sum_j w[c][j] * in[t - (taps-1) + j][c]) over the token's own sequence,
//                        rows before the step's first token come from the sequence's state (zeros at its start);
//                        then the state takes the last taps-1 inputs.  One token per sequence: one launch does both.
//   tb_mamba2_scan       per head h (group g = h / (heads / groups)), with dt = softplus(dt_raw + dt_bias):
//                          S <- exp(-exp(A_log[h]) dt) S + dt * x_t B_t^T      S is [P][N]
//                          y_t = S C_t + D[h] x_t
//                        sequential over a sequence's tokens, S read from and written back to the state.
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
    const void* proj; long long proj_stride;      // [tokens][inner + channels + heads], compute dtype
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
// The recurrence.  A CTA of 128 threads owns (sequence, head, 16 values of P): thread (pl, ns) holds the NPT states
// S[p][ns * NPT .. (ns + 1) * NPT) in registers (eight threads share a p and add their parts of y by shuffles).  B and
// C of TT tokens at a time are staged in shared memory.
#define SCAN_NS 8
#define SCAN_PT 16
#define SCAN_TT 16

template <typename T, typename TW, int NPT>
__global__ void __launch_bounds__(SCAN_NS * SCAN_PT) mamba2_scan_kernel(Mamba2Args a) {
    pdl_launch_dependents();
    extern __shared__ float sh[];                                    // [TT][2][N] B and C, then [TT][PT] x, then [TT][2] dt and decay
    const int N = a.N, P = a.P, H = a.heads;
    const int inner = H * P, ch = inner + 2 * a.groups * N;
    const int b = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * SCAN_PT;
    const int g = h / (H / a.groups);
    const int ns = threadIdx.x % SCAN_NS, pl = threadIdx.x / SCAN_NS;
    const int p = p0 + pl;
    const int n0 = ns * NPT;
    float* sBC = sh;
    float* sx = sh + SCAN_TT * 2 * N;
    float* sdt = sx + SCAN_TT * SCAN_PT;
    const float A = -expf(to_f<TW>(((const TW*)a.A_log)[h]));
    const float Dh = to_f<TW>(((const TW*)a.D)[h]);
    const float dtb = to_f<TW>(((const TW*)a.dt_bias)[h]);
    pdl_wait();
    const int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    float* S = a.state + (size_t)a.slot_ids[b] * a.state_stride + ((size_t)h * P + (p < P ? p : 0)) * N;
    float s[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) s[k] = (p < P && n0 + k < N) ? S[n0 + k] : 0.f;
    const T* xbc = (const T*)a.xbc;
    const T* proj = (const T*)a.proj;
    for (int tb = s0; tb < s1; tb += SCAN_TT) {
        const int nt = min(SCAN_TT, s1 - tb);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 2 * N; i += blockDim.x) {
            const int tt = i / (2 * N), r = i % (2 * N);             // r < N: B, else C
            const int col = inner + (r < N ? g * N + r : a.groups * N + g * N + (r - N));
            sBC[i] = to_f<T>(xbc[(size_t)(tb + tt) * ch + col]);
        }
        for (int i = threadIdx.x; i < nt * SCAN_PT; i += blockDim.x) {
            const int tt = i / SCAN_PT, pp = p0 + i % SCAN_PT;
            sx[i] = pp < P ? to_f<T>(xbc[(size_t)(tb + tt) * ch + h * P + pp]) : 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += blockDim.x) {
            const float dt = softplus_f(to_f<T>(proj[(size_t)(tb + i) * a.proj_stride + inner + ch + h]) + dtb);
            sdt[2 * i] = dt;
            sdt[2 * i + 1] = expf(A * dt);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float dt = sdt[2 * tt], dec = sdt[2 * tt + 1];
            const float x = sx[tt * SCAN_PT + pl];
            const float dx = dt * x;
            const float* Bt = sBC + (size_t)tt * 2 * N;
            const float* Ct = Bt + N;
            float y = 0.f;
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                if (n0 + k < N) {
                    s[k] = dec * s[k] + dx * Bt[n0 + k];
                    y += s[k] * Ct[n0 + k];
                }
            }
#pragma unroll
            for (int o = SCAN_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0 && p < P) a.y[(size_t)(tb + tt) * inner + h * P + p] = y + Dh * x;
        }
    }
    if (p < P) {
#pragma unroll
        for (int k = 0; k < NPT; k++) if (n0 + k < N) S[n0 + k] = s[k];
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

#define DISPATCH2(ct, cw, ...)                                                             \
    do {                                                                                   \
        if ((ct) == TB_F32 && (cw) == TB_F32) { typedef float T; typedef float TW; __VA_ARGS__; }        \
        else if ((ct) == TB_BF16 && (cw) == TB_BF16) { typedef bf16 T; typedef bf16 TW; __VA_ARGS__; }   \
        else if ((ct) == TB_BF16 && (cw) == TB_F32) { typedef bf16 T; typedef float TW; __VA_ARGS__; }   \
        else if ((ct) == TB_F32 && (cw) == TB_BF16) { typedef float T; typedef bf16 TW; __VA_ARGS__; }   \
        else return tb_refuse("mamba2: unknown dtype codes %d %d", (ct), (cw));              \
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

extern "C" int tb_mamba2_scan(const Mamba2Args* args, int dtype, int w_dtype, cudaStream_t stream) {
    Mamba2Args a = *args;
    if (a.n_tokens <= 0) return 0;
    if (check(a)) return -1;
    const dim3 grid((a.P + SCAN_PT - 1) / SCAN_PT, a.heads, a.batch);
    if (grid.y > 65535 || grid.z > 65535) return tb_refuse("mamba2: too many heads or sequences for one launch");
    const size_t smem = (size_t)(SCAN_TT * 2 * a.N + SCAN_TT * SCAN_PT + SCAN_TT * 2) * sizeof(float);
    const int npt = (a.N + SCAN_NS - 1) / SCAN_NS;
#define SCAN(NPT_) DISPATCH2(dtype, w_dtype, tb_launch(mamba2_scan_kernel<T, TW, NPT_>, dim3(grid), dim3(SCAN_NS * SCAN_PT), smem, stream, a))
    if (npt <= 2) SCAN(2); else if (npt <= 4) SCAN(4); else if (npt <= 8) SCAN(8); else if (npt <= 16) SCAN(16); else SCAN(32);
#undef SCAN
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
    DISPATCH2(dtype, w_dtype, tb_launch(mamba2_gate_norm_kernel<T, TW>, dim3(a.n_tokens, a.norm_groups), dim3(threads), 0, stream, a));
    return tb_launch_status();
}
