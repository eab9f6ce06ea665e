// Attention over cached latent rows: the kernels that are particular to it.
//
// A token leaves one row in the cache: [c (C numbers) | r (R numbers)], c a normed latent from which every
// head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c) and r a rotated key part that all
// heads share.  A head's score of query (a | b) against a token is  a . (Uk_h c) + b . r  =  (Uk_h^T a) . c + b . r,
// so with the query mapped once to q' = (Uk_h^T a | b) every head reads the same rows (keys of C + R numbers,
// values their first C numbers) and its output Uv_h (sum_j p_j c_j) is mapped back afterwards.
//
//   tb_latent_rows     from the 32-bit partial sums of the down projection: c = rms-normed first C columns
//                      times a weight, r = the last R columns rotated at the token's position (rotate-half
//                      pairing over the first rot_dims of them); the row goes to the paged cache and to a
//                      packed matrix; all arithmetic 32-bit, the row rounded once
//   tb_head_linear     y[t, h, :] = W[h] x[t, h, :] for per-head matrices W [heads][out][in]
//   tb_latent_decode   one query per sequence and head against the cached rows, the key range cut into
//                      splits; softmax with a sink: the denominator also holds exp(sink_h), which has no
//                      key and no value; partial (max, sum, o) per split are folded in split order
#include "common.cuh"

TB_EXPORT_ERROR()

struct LatentRowsArgs {
    const float* dkv; int splits; long long split_stride;     // [splits][T][C + R]
    const float* norm_w; float eps;                            // [C]
    const float* inv_freq; int rot_dims;                       // [rot_dims / 2]
    int C, R, n_tokens;
    const int* positions; const int* token_seq;
    const int* page_table; int pt_stride; int page_rows;
    void* pool;                                                // [pages][page_rows][C + R]
    void* rows;                                                // [T][C + R]
};

template <typename T>
__global__ void __launch_bounds__(128) latent_rows_kernel(LatentRowsArgs a) {
    pdl_launch_dependents();
    extern __shared__ float row_s[];
    __shared__ float red[33];
    const int t = blockIdx.x, W = a.C + a.R;
    pdl_wait();
    float sq = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < a.splits; s++) v += a.dkv[(size_t)s * a.split_stride + (size_t)t * W + c];
        row_s[c] = v;
        if (c < a.C) sq = fmaf(v, v, sq);
    }
    const float rinv = 1.f / sqrtf(block_sum(sq, red) / (float)a.C + a.eps);     // its barriers also publish row_s
    const int pos = a.positions[t];
    const int page = a.page_table[(size_t)a.token_seq[t] * a.pt_stride + pos / a.page_rows];
    T* cache = (T*)a.pool + ((size_t)page * a.page_rows + pos % a.page_rows) * W;
    T* out = (T*)a.rows + (size_t)t * W;
    const int half = a.rot_dims / 2;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float v;
        if (c < a.C) {
            v = row_s[c] * rinv * a.norm_w[c];
        } else {
            const int i = c - a.C;
            if (i < half) {
                float sn, cs; sincosf((float)pos * a.inv_freq[i], &sn, &cs);
                v = row_s[c] * cs - row_s[c + half] * sn;
            } else if (i < 2 * half) {
                float sn, cs; sincosf((float)pos * a.inv_freq[i - half], &sn, &cs);
                v = row_s[c] * cs + row_s[c - half] * sn;
            } else {
                v = row_s[c];
            }
        }
        const T r = from_f<T>(v);
        cache[c] = r; out[c] = r;
    }
}

// ---------------------------------------------------------------------------
constexpr int HL_TOK = 8;

template <typename T>
__global__ void __launch_bounds__(128) head_linear_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w,
                                                          T* __restrict__ y, long long y_stride, int n_tokens, int in, int out) {
    pdl_launch_dependents();
    extern __shared__ float x_s[];                      // [HL_TOK][in]
    const int h = blockIdx.y, t0 = blockIdx.x * HL_TOK;
    const int nt = min(HL_TOK, n_tokens - t0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < HL_TOK * in; i += blockDim.x) {
        const int tt = i / in, c = i % in;
        x_s[i] = tt < nt ? to_f<T>(x[(size_t)(t0 + tt) * x_stride + (size_t)h * in + c]) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (size_t)h * out * in;
    for (int o = blockIdx.z * nwarp + warp; o < out; o += gridDim.z * nwarp) {
        float acc[HL_TOK];
#pragma unroll
        for (int tt = 0; tt < HL_TOK; tt++) acc[tt] = 0.f;
        for (int c = lane; c < in; c += 32) {
            const float wv = to_f<T>(wh[(size_t)o * in + c]);
#pragma unroll
            for (int tt = 0; tt < HL_TOK; tt++) acc[tt] = fmaf(wv, x_s[tt * in + c], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_TOK; tt++) {
            const float s = warp_sum(acc[tt]);
            if (lane == 0 && tt < nt) y[(size_t)(t0 + tt) * y_stride + (size_t)h * out + o] = from_f<T>(s);
        }
    }
}

extern "C" int tb_head_linear(const void* x, long long x_stride, const void* w, void* y, long long y_stride, int dtype,
                              int n_tokens, int heads, int in, int out, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || in <= 0 || out <= 0 || in > 1536)
        return tb_refuse("head_linear: heads=%d in=%d out=%d (in at most 1536)", heads, in, out);
    const int zs = (out + 63) / 64 < 64 ? (out + 63) / 64 : 64;
    dim3 grid((n_tokens + HL_TOK - 1) / HL_TOK, heads, zs);
    TB_DISPATCH_1(dtype, T, tb_launch(head_linear_kernel<T>, dim3(grid), dim3(128), (size_t)HL_TOK * in * sizeof(float), stream,
                                      (const T*)x, x_stride, (const T*)w, (T*)y, y_stride, n_tokens, in, out));
    return tb_launch_status();
}

extern "C" int tb_latent_rows(const LatentRowsArgs* args, int dtype, cudaStream_t stream) {
    const LatentRowsArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.C <= 0 || a.R < 0 || a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.R || a.page_rows <= 0)
        return tb_refuse("latent_rows: C=%d R=%d rot_dims=%d page_rows=%d", a.C, a.R, a.rot_dims, a.page_rows);
    TB_DISPATCH_1(dtype, T, tb_launch(latent_rows_kernel<T>, dim3(a.n_tokens), dim3(128), (size_t)(a.C + a.R) * sizeof(float), stream, a));
    return tb_launch_status();
}

// ---------------------------------------------------------------------------
struct LatentDecodeArgs {
    const void* q; long long q_stride;                 // [batch] rows of heads * (C + R): the mapped queries
    const void* pool;                                  // [pages][page_rows][C + R]
    const int* page_table; int pt_stride; int page_rows;
    const int* len_after;                              // [batch] rows in the cache, the new token's included
    const float* sink;                                 // [heads] or null
    void* out; long long out_stride;                   // [batch] rows of heads * out_dim; the first C of a head are written
    float* partial;                                    // [batch][heads][splits][C + 2] when splits > 1
    int heads, C, R, out_dim, n_splits;
    float scale;
};

template <int NC>
struct LatAcc {
    float m, l, o[NC];
    __device__ void init() { m = -INFINITY; l = 0.f;
#pragma unroll
        for (int c = 0; c < NC; c++) o[c] = 0.f; }
};

template <typename T, int NC>
__global__ void __launch_bounds__(128) latent_decode_kernel(LatentDecodeArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const int KD = a.C + a.R, C = a.C;
    float* q_s = smem;                                 // [KD]
    float* red = smem + KD;                            // [nwarp][C + 2]
    pdl_wait();
    const T* qrow = (const T*)a.q + (size_t)b * a.q_stride + (size_t)h * KD;
    for (int e = threadIdx.x; e < KD; e += blockDim.x) q_s[e] = to_f<T>(qrow[e]);
    __syncthreads();
    const int len = a.len_after[b];
    int per = (len + a.n_splits - 1) / a.n_splits;
    per = (per + 31) & ~31;
    const int beg = split * per, end = min(len, beg + per);
    const int* pt = a.page_table + (size_t)b * a.pt_stride;

    LatAcc<NC> acc; acc.init();
    for (int j0 = beg + warp * 32; j0 < end; j0 += nwarp * 32) {
        const int j = j0 + lane;
        const bool valid = j < end;
        const T* krow = nullptr;
        float s = -INFINITY;
        if (valid) {
            krow = (const T*)a.pool + ((size_t)pt[j / a.page_rows] * a.page_rows + (j % a.page_rows)) * KD;
            float d = 0.f;
            for (int e = 0; e < KD; e++) d = fmaf(q_s[e], to_f<T>(krow[e]), d);
            s = d * a.scale;
        }
        const float cm = warp_max(s);
        const float m_new = fmaxf(acc.m, cm);
        const float corr = (acc.m == -INFINITY) ? 0.f : expf(acc.m - m_new);
        const float p = valid ? expf(s - m_new) : 0.f;
        acc.l = acc.l * corr + warp_sum(p);
        acc.m = m_new;
#pragma unroll
        for (int c = 0; c < NC; c++) acc.o[c] *= corr;
        for (int jj = 0; jj < 32; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)krow, jj);
            if (pj == 0.f) continue;
            const T* v = (const T*)(uintptr_t)vp;
#pragma unroll
            for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < C) acc.o[c] = fmaf(pj, to_f<T>(v[d]), acc.o[c]); }
        }
    }
    float* mine = red + (size_t)warp * (C + 2);
    if (lane == 0) { mine[C] = acc.m; mine[C + 1] = acc.l; }
#pragma unroll
    for (int c = 0; c < NC; c++) { const int d = lane + 32 * c; if (d < C) mine[d] = acc.o[c]; }
    __syncthreads();
    const float sink = (a.sink != nullptr) ? a.sink[h] : -INFINITY;
    float M = (a.n_splits == 1) ? sink : -INFINITY;
    for (int w = 0; w < nwarp; w++) M = fmaxf(M, red[(size_t)w * (C + 2) + C]);
    float L = 0.f;
    for (int w = 0; w < nwarp; w++) {
        const float mw = red[(size_t)w * (C + 2) + C];
        if (mw != -INFINITY) L += red[(size_t)w * (C + 2) + C + 1] * expf(mw - M);
    }
    if (a.n_splits == 1 && sink != -INFINITY) L += expf(sink - M);
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < nwarp; w++) {
            const float mw = red[(size_t)w * (C + 2) + C];
            if (mw != -INFINITY) o += red[(size_t)w * (C + 2) + d] * expf(mw - M);
        }
        if (a.n_splits == 1) ((T*)a.out)[(size_t)b * a.out_stride + (size_t)h * a.out_dim + d] = from_f<T>(o / L);
        else a.partial[(((size_t)b * a.heads + h) * a.n_splits + split) * (C + 2) + d] = o;
    }
    if (a.n_splits > 1 && threadIdx.x == 0) {
        float* p = a.partial + (((size_t)b * a.heads + h) * a.n_splits + split) * (C + 2);
        p[C] = M; p[C + 1] = L;
    }
}

template <typename T>
__global__ void latent_combine_kernel(LatentDecodeArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, C = a.C, n = a.n_splits;
    const float* p = a.partial + ((size_t)b * a.heads + h) * n * (C + 2);
    const float sink = (a.sink != nullptr) ? a.sink[h] : -INFINITY;
    float M = sink;
    for (int s = 0; s < n; s++) M = fmaxf(M, p[(size_t)s * (C + 2) + C]);
    float L = (sink != -INFINITY) ? expf(sink - M) : 0.f;
    for (int s = 0; s < n; s++) {
        const float ms = p[(size_t)s * (C + 2) + C];
        if (ms != -INFINITY) L += p[(size_t)s * (C + 2) + C + 1] * expf(ms - M);
    }
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n; s++) {
            const float ms = p[(size_t)s * (C + 2) + C];
            if (ms != -INFINITY) o += p[(size_t)s * (C + 2) + d] * expf(ms - M);
        }
        ((T*)a.out)[(size_t)b * a.out_stride + (size_t)h * a.out_dim + d] = from_f<T>(o / L);
    }
}

extern "C" int tb_latent_decode(const LatentDecodeArgs* args, int dtype, int batch, cudaStream_t stream) {
    if (batch <= 0) return 0;
    const LatentDecodeArgs& a = *args;
    if (a.heads <= 0 || a.heads > 65535 || a.C <= 0 || a.R < 0 || a.C > 512 || a.out_dim < a.C)
        return tb_refuse("latent_decode: heads=%d C=%d R=%d out_dim=%d (C at most 512)", a.heads, a.C, a.R, a.out_dim);
    if (a.n_splits < 1 || a.n_splits > 65535 || (a.n_splits > 1 && a.partial == nullptr))
        return tb_refuse("latent_decode: n_splits=%d needs scratch", a.n_splits);
    const int warps = 4;
    const size_t smem = ((size_t)(a.C + a.R) + (size_t)warps * (a.C + 2)) * sizeof(float);
    int nc = 1;
    while (nc * 32 < a.C) nc <<= 1;
    dim3 grid(batch, a.heads, a.n_splits);
#define LAT_DEC(N) TB_DISPATCH_1(dtype, T, tb_launch(latent_decode_kernel<T, N>, dim3(grid), dim3(warps * 32), smem, stream, a))
    switch (nc) {
    case 1: LAT_DEC(1); break;
    case 2: LAT_DEC(2); break;
    case 4: LAT_DEC(4); break;
    case 8: LAT_DEC(8); break;
    default: LAT_DEC(16); break;
    }
    int st = tb_launch_status();
    if (st || a.n_splits == 1) return st;
    TB_DISPATCH_1(dtype, T, tb_launch(latent_combine_kernel<T>, dim3(batch, a.heads), dim3(128), 0, stream, a));
    return tb_launch_status();
}
