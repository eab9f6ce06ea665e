// Gated linear attention: everything between the input products and the output product.
//
// Per head, with key channels d and value channels v, for the tokens of a sequence in order:
//     S[d][v] <- decay_t[d] * S[d][v] + k_t[d] * v_t[v];      o_t[v] = sum_d S[d][v] * q_t[d]
// where decay_t[d] = sigmoid(z_t[d])^(1/tau) and z_t = A2 (A1 x_t) + bias (a product of low rank).
// Then every head's o_t is divided by its root mean square over v (+ eps inside the root), multiplied
// by a weight shared by the heads and by silu(g_t).
//
//   tb_gla_decay      z from the 32-bit partial sums of A1 x, the decay as exp(-softplus(-z) / tau)
//   tb_gla_scan       the recurrence; the state S of every sequence lives in a 32-bit row addressed by
//                     slot, is read at the start of the step's tokens and written back at their end,
//                     so a step of whole prompts and a step of one token each are the same kernel
//   tb_gla_gate_norm  the unit norm, the weight and the gate; output in the activations' dtype
//
// 32-bit throughout: z, the decay, the state, o and the norm.  q, k, v and g arrive in the activations'
// dtype (they are products) and are widened on the way in.
//
// The scan: one CTA = 64 value channels of one head of one sequence (or of a chunk in time of it), eight warps
// that each own an eighth of the key channels; a thread keeps its part of two columns of S in registers.  q, k
// and the decay of eight tokens at a time are staged in shared memory (every thread of a warp reads the same
// 16-byte word: a broadcast that serves both columns), the next eight are on their way through registers
// meanwhile; the warps' partial outputs of a tile meet in shared memory once per tile.
#include "common.cuh"

TB_EXPORT_ERROR()

struct GlaArgs {
    const void* proj; long long proj_stride;          // [T] rows of q (H*D), k (H*D), v (H*V), g (H*V)
    const float* a1; int a1_splits; long long a1_split_stride; int rank;   // [splits][T][rank]
    const float* a2; const float* a2_bias;            // [H*D][rank], [H*D]
    float inv_tau, q_scale;
    const float* norm_w; float eps;                   // [V]
    float* state; long long state_stride;             // [slots][H*D*V]
    const int* seq_start; const int* token_seq; const int* slot_ids;
    float* decay;                                     // [T][H*D] scratch
    float* y;                                         // [T][H*V] scratch
    void* out;                                        // [T][H*V]
    int heads, D, V, batch, n_tokens;
    // long prompts cut into chunks in time that run side by side (0 chunks: one CTA walks a whole sequence)
    float* chunk_state;                               // [batch][n_chunks][H*D*V]: a chunk's end state from zero, then its start state
    float* chunk_decay;                               // [batch][n_chunks][H*D]: the product of the chunk's decays
    int chunk_len, n_chunks;
};

constexpr int GLA_DECAY_TOK = 32;

// 32 tokens and 256 channels per CTA: a thread owns a channel, keeps the 32 sums in registers and reads its row of A2 once.
__global__ void __launch_bounds__(256) gla_decay_kernel(GlaArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float low_s[];                  // [32][rank]: A1 x of these tokens
    const int t0 = blockIdx.x * GLA_DECAY_TOK, nt = min(GLA_DECAY_TOK, a.n_tokens - t0);
    const int HD = a.heads * a.D;
    for (int i = threadIdx.x; i < GLA_DECAY_TOK * a.rank; i += blockDim.x) {
        const int tt = i / a.rank, r = i % a.rank;
        float v = 0.f;
        if (tt < nt)
            for (int s = 0; s < a.a1_splits; s++) v += a.a1[(size_t)s * a.a1_split_stride + (size_t)(t0 + tt) * a.rank + r];
        low_s[i] = v;
    }
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= HD) return;
    float z[GLA_DECAY_TOK];
    const float bias = a.a2_bias[c];
#pragma unroll
    for (int tt = 0; tt < GLA_DECAY_TOK; tt++) z[tt] = 0.f;
    const float* w = a.a2 + (size_t)c * a.rank;
    for (int r = 0; r < a.rank; r++) {
        const float wr = w[r];
#pragma unroll
        for (int tt = 0; tt < GLA_DECAY_TOK; tt++) z[tt] = fmaf(wr, low_s[tt * a.rank + r], z[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < GLA_DECAY_TOK; tt++) {
        if (tt >= nt) break;
        const float x = -(z[tt] + bias);               // log sigmoid(z) = -softplus(-z)
        const float sp = x > 20.f ? x : log1pf(expf(x));
        a.decay[(size_t)(t0 + tt) * HD + c] = expf(-sp * a.inv_tau);
    }
}

constexpr int GLA_TT = 8;          // tokens per tile
constexpr int GLA_WARPS = 8;       // slices of the key channels

// MODE 0: a sequence from the state its slot holds to the state it leaves there, with outputs.
// MODE 1: a chunk from a zero state, without outputs: its end state and the product of its decays (for the fold).
// MODE 2: a chunk from the start state the fold left, with outputs; the last chunk leaves the sequence's state.
constexpr int GLA_VT = 64;         // value channels per CTA: two per thread, so that a word of q, k or the decay serves two updates

template <typename T, int DPT, int MODE>
__global__ void __launch_bounds__(GLA_WARPS * 32, 2) gla_scan_kernel(GlaArgs a) {
    pdl_launch_dependents();
    constexpr int DP = DPT * GLA_WARPS;                // key channels, padded
    constexpr int PER = (GLA_TT * DP + GLA_WARPS * 32 - 1) / (GLA_WARPS * 32);   // staged (token, channel) places per thread
    __shared__ __align__(16) float q_s[GLA_TT][DP], k_s[GLA_TT][DP], d_s[GLA_TT][DP];
    __shared__ float v_s[GLA_TT][GLA_VT];
    __shared__ float part_s[GLA_TT][GLA_WARPS][GLA_VT];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y;
    const int b = MODE == 0 ? blockIdx.z : blockIdx.z / a.n_chunks;
    const int chunk = MODE == 0 ? 0 : blockIdx.z % a.n_chunks;
    const int D = a.D, V = a.V, HD = a.heads * D, HV = a.heads * V;
    const int v0 = blockIdx.x * GLA_VT;
    const int vc[2] = {v0 + lane, v0 + lane + 32};
    const bool v_ok[2] = {vc[0] < V, vc[1] < V};
    pdl_wait();
    int s0 = a.seq_start[b], s1 = a.seq_start[b + 1];
    const int seq_end = s1;
    if (MODE != 0) { s0 = min(s1, s0 + chunk * a.chunk_len); s1 = min(s1, s0 + a.chunk_len); }
    float* st = a.state + (size_t)a.slot_ids[b] * a.state_stride + (size_t)h * D * V;
    float* cst = MODE == 0 ? nullptr : a.chunk_state + ((size_t)b * a.n_chunks + chunk) * a.heads * D * V + (size_t)h * D * V;
    float S[2][DPT], P[MODE == 1 ? DPT : 1];
#pragma unroll
    for (int j = 0; j < DPT; j++) {
        const int d = warp * DPT + j;
        const float* from = MODE == 2 ? cst : st;
#pragma unroll
        for (int c = 0; c < 2; c++) S[c][j] = (MODE != 1 && d < D && v_ok[c]) ? from[(size_t)d * V + vc[c]] : 0.f;
        if (MODE == 1) P[j] = 1.f;
    }
    const T* proj = (const T*)a.proj;
    // a tile's q, k, decay and v travel through registers: the next tile's loads are in flight while this one is computed
    float rq[PER], rk[PER], rd[PER], rv[2];
    auto fetch = [&](int t0) {
        const int nt = min(GLA_TT, s1 - t0);
#pragma unroll
        for (int u = 0; u < PER; u++) {
            const int i = threadIdx.x + u * GLA_WARPS * 32;
            const int tt = i / DP, d = i % DP;
            rq[u] = 0.f; rk[u] = 0.f; rd[u] = 1.f;
            if (i < GLA_TT * DP && tt < nt && d < D) {
                const T* row = proj + (size_t)(t0 + tt) * a.proj_stride;
                if (MODE != 1) rq[u] = to_f<T>(row[h * D + d]) * a.q_scale;
                rk[u] = to_f<T>(row[HD + h * D + d]);
                rd[u] = a.decay[(size_t)(t0 + tt) * HD + h * D + d];
            }
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {                  // 8 tokens x 64 channels = 2 per thread
            const int i = threadIdx.x + u * GLA_WARPS * 32;
            const int tt = i / GLA_VT, c = v0 + i % GLA_VT;
            rv[u] = (tt < nt && c < V) ? to_f<T>(proj[(size_t)(t0 + tt) * a.proj_stride + 2 * HD + h * V + c]) : 0.f;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < PER; u++) {
            const int i = threadIdx.x + u * GLA_WARPS * 32;
            if (i < GLA_TT * DP) { (&q_s[0][0])[i] = rq[u]; (&k_s[0][0])[i] = rk[u]; (&d_s[0][0])[i] = rd[u]; }
        }
#pragma unroll
        for (int u = 0; u < 2; u++) (&v_s[0][0])[threadIdx.x + u * GLA_WARPS * 32] = rv[u];
    };
    if (s0 < s1) { fetch(s0); stash(); }
    __syncthreads();
    for (int t0 = s0; t0 < s1; t0 += GLA_TT) {
        const int nt = min(GLA_TT, s1 - t0);
        const bool more = t0 + GLA_TT < s1;
        if (more) fetch(t0 + GLA_TT);
        for (int tt = 0; tt < nt; tt++) {
            const float va = v_s[tt][lane], vb = v_s[tt][lane + 32];
            float acc_a = 0.f, acc_b = 0.f;
            if constexpr (DPT % 4 == 0) {
                const float4* d4 = reinterpret_cast<const float4*>(&d_s[tt][warp * DPT]);
                const float4* k4 = reinterpret_cast<const float4*>(&k_s[tt][warp * DPT]);
                const float4* q4 = reinterpret_cast<const float4*>(&q_s[tt][warp * DPT]);
#pragma unroll
                for (int j4 = 0; j4 < DPT / 4; j4++) {
                    const float4 dd = d4[j4], kk = k4[j4];
                    const float dv[4] = {dd.x, dd.y, dd.z, dd.w}, kv[4] = {kk.x, kk.y, kk.z, kk.w};
                    float qv[4] = {0.f, 0.f, 0.f, 0.f};
                    if (MODE != 1) { const float4 qq = q4[j4]; qv[0] = qq.x; qv[1] = qq.y; qv[2] = qq.z; qv[3] = qq.w; }
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int j = j4 * 4 + e;
                        S[0][j] = fmaf(dv[e], S[0][j], kv[e] * va);
                        S[1][j] = fmaf(dv[e], S[1][j], kv[e] * vb);
                        if (MODE == 1) P[j] *= dv[e];
                        else { acc_a = fmaf(S[0][j], qv[e], acc_a); acc_b = fmaf(S[1][j], qv[e], acc_b); }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < DPT; j++) {
                    const int d = warp * DPT + j;
                    const float dec = d_s[tt][d], kk = k_s[tt][d];
                    S[0][j] = fmaf(dec, S[0][j], kk * va);
                    S[1][j] = fmaf(dec, S[1][j], kk * vb);
                    if (MODE == 1) P[j] *= dec;
                    else { acc_a = fmaf(S[0][j], q_s[tt][d], acc_a); acc_b = fmaf(S[1][j], q_s[tt][d], acc_b); }
                }
            }
            if (MODE != 1) { part_s[tt][warp][lane] = acc_a; part_s[tt][warp][lane + 32] = acc_b; }
        }
        __syncthreads();                               // every warp is done with the tile; the partial outputs are complete
        if (MODE != 1) {
            const int tt = warp;                       // 8 warps = the tile's 8 tokens
            if (tt < nt) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    float o = 0.f;
#pragma unroll
                    for (int w = 0; w < GLA_WARPS; w++) o += part_s[tt][w][lane + 32 * c];
                    if (v_ok[c]) a.y[(size_t)(t0 + tt) * HV + h * V + vc[c]] = o;
                }
            }
        }
        if (more) stash();
        __syncthreads();                               // the next tile is in shared memory; the partial outputs are free again
    }
    if (MODE == 2 && s1 != seq_end) return;            // only the chunk that holds the sequence's end leaves its state
    if (MODE == 2 && s0 == s1 && chunk != 0) return;   // (an empty chunk after the end: the one before it did)
#pragma unroll
    for (int j = 0; j < DPT; j++) {
        const int d = warp * DPT + j;
        float* to = MODE == 1 ? cst : st;
#pragma unroll
        for (int c = 0; c < 2; c++)
            if (d < D && v_ok[c]) to[(size_t)d * V + vc[c]] = S[c][j];
        if (MODE == 1 && d < D && blockIdx.x == 0 && lane == 0)
            a.chunk_decay[((size_t)b * a.n_chunks + chunk) * a.heads * D + (size_t)h * D + d] = P[j];
    }
}

// Start states of the chunks from their end states: S_start[0] = the slot's state, S_start[c+1] = P_c S_start[c] + E_c,
// element by element; chunk_state[c] is turned from E_c into S_start[c] in place.
__global__ void gla_fold_kernel(GlaArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int D = a.D, V = a.V;
    const long long per = (long long)a.heads * D * V;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per * a.batch) return;
    const int b = (int)(i / per);
    const long long e = i % per;                      // (h, d, v)
    const long long hd = e / V;                       // h * D + d
    float S = a.state[(size_t)a.slot_ids[b] * a.state_stride + e];
    float* cs = a.chunk_state + (size_t)b * a.n_chunks * per + e;
    const float* cd = a.chunk_decay + (size_t)b * a.n_chunks * a.heads * D + hd;
    for (int c0 = 0; c0 < a.n_chunks; c0 += 8) {       // eight chunks' end states and decays on their way together
        float E[8], P[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const bool in = c0 + u < a.n_chunks;
            E[u] = in ? cs[(size_t)(c0 + u) * per] : 0.f;
            P[u] = in ? cd[(size_t)(c0 + u) * a.heads * D] : 1.f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (c0 + u < a.n_chunks) {
                cs[(size_t)(c0 + u) * per] = S;
                S = fmaf(P[u], S, E[u]);
            }
        }
    }
}

template <typename T>
__global__ void gla_gate_norm_kernel(GlaArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)a.n_tokens * a.heads) return;
    const int t = (int)(item / a.heads), h = (int)(item % a.heads);
    const int V = a.V, HV = a.heads * V, HD = a.heads * a.D;
    const float* y = a.y + (size_t)t * HV + (size_t)h * V;
    float sq = 0.f;
    for (int v = lane; v < V; v += 32) sq = fmaf(y[v], y[v], sq);
    const float r = 1.f / sqrtf(warp_sum(sq) / (float)V + a.eps);
    const T* g = (const T*)a.proj + (size_t)t * a.proj_stride + 2 * HD + HV + (size_t)h * V;
    T* o = (T*)a.out + (size_t)t * HV + (size_t)h * V;
    for (int v = lane; v < V; v += 32) {
        const float gv = to_f<T>(g[v]);
        o[v] = from_f<T>(y[v] * r * a.norm_w[v] * (gv / (1.f + expf(-gv))));
    }
}

static int check(const GlaArgs& a) {
    if (a.heads <= 0 || a.D <= 0 || a.V <= 0 || a.rank <= 0) return tb_refuse("gla: heads=%d D=%d V=%d rank=%d", a.heads, a.D, a.V, a.rank);
    if (a.D > 256) return tb_refuse("gla: %d key channels per head; the scan keeps up to 256", a.D);
    if (a.heads > 65535 || a.batch > 65535) return tb_refuse("gla: %d heads x %d sequences exceed one launch", a.heads, a.batch);
    return 0;
}

extern "C" int tb_gla_decay(const GlaArgs* args, cudaStream_t stream) {
    if (args->n_tokens <= 0) return 0;
    if (check(*args)) return -1;
    if (args->rank > 256) return tb_refuse("gla: a decay of rank %d; the kernel takes up to 256", args->rank);
    const int HD = args->heads * args->D;
    tb_launch(gla_decay_kernel, dim3((args->n_tokens + GLA_DECAY_TOK - 1) / GLA_DECAY_TOK, (HD + 255) / 256), dim3(256),
              (size_t)GLA_DECAY_TOK * args->rank * sizeof(float), stream, *args);
    return tb_launch_status();
}

extern "C" int tb_gla_scan(const GlaArgs* args, int dtype, cudaStream_t stream) {
    if (args->n_tokens <= 0 || args->batch <= 0) return 0;
    if (check(*args)) return -1;
    const GlaArgs& a = *args;
    int dpt = 1;
    while (dpt * GLA_WARPS < a.D) dpt <<= 1;
    const bool chunks = a.n_chunks > 1;
    if (chunks && (a.chunk_len <= 0 || a.chunk_state == nullptr || a.chunk_decay == nullptr || (long long)a.batch * a.n_chunks > 65535))
        return tb_refuse("gla: %d chunks of %d tokens need their scratch (and batch x chunks <= 65535)", a.n_chunks, a.chunk_len);
    dim3 grid((a.V + GLA_VT - 1) / GLA_VT, a.heads, chunks ? a.batch * a.n_chunks : a.batch);
#define GLA_SCAN_M(N, M) TB_DISPATCH_1(dtype, T, tb_launch(gla_scan_kernel<T, N, M>, dim3(grid), dim3(GLA_WARPS * 32), 0, stream, a))
#define GLA_SCAN(N) do { if (mode == 0) GLA_SCAN_M(N, 0); else if (mode == 1) GLA_SCAN_M(N, 1); else GLA_SCAN_M(N, 2); } while (0)
    for (int pass = 0; pass < (chunks ? 3 : 1); pass++) {
        if (chunks && pass == 1) {
            const long long n = (long long)a.batch * a.heads * a.D * a.V;
            tb_launch(gla_fold_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, a);
        } else {
            const int mode = chunks ? (pass == 0 ? 1 : 2) : 0;
            switch (dpt) {
            case 1: GLA_SCAN(1); break;
            case 2: GLA_SCAN(2); break;
            case 4: GLA_SCAN(4); break;
            case 8: GLA_SCAN(8); break;
            case 16: GLA_SCAN(16); break;
            default: GLA_SCAN(32); break;
            }
        }
        const int st = tb_launch_status();
        if (st) return st;
    }
    return 0;
}

// How a step of whole prompts is cut in time: chunks of at least 64 tokens, as many as fill the GPU once (two CTAs an SM)
// and no more, so that no CTA waits for a second round.
extern "C" int tb_gla_plan(int heads, int V, int batch, int max_seq_len, int sms, int* chunk_len) {
    const long long ctas = (long long)((V + GLA_VT - 1) / GLA_VT) * heads * batch;
    int want = (int)((2LL * sms) / ctas);
    int most = max_seq_len / 64;
    if (want > most) want = most;
    if (want <= 1) { *chunk_len = 0; return 1; }
    int len = (max_seq_len + want - 1) / want;
    len = (len + GLA_TT - 1) / GLA_TT * GLA_TT;
    *chunk_len = len;
    return (max_seq_len + len - 1) / len;
}

extern "C" int tb_gla_gate_norm(const GlaArgs* args, int dtype, cudaStream_t stream) {
    if (args->n_tokens <= 0) return 0;
    if (check(*args)) return -1;
    const long long items = (long long)args->n_tokens * args->heads;
    TB_DISPATCH_1(dtype, T, tb_launch(gla_gate_norm_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, *args));
    return tb_launch_status();
}
