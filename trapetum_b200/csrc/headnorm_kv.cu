// Per-head unit norm of q and k, query temperature, and the write of k and v into the paged cache.
//
// For mixers whose positions do not enter through a rotation.  The input is the q/k(/v) product as 32-bit
// partial sums [splits][tokens][in_width] (added here in split order); everything is computed in 32-bit and
// rounded once, on the way out:
//
//   q_h <- q_h / sqrt(mean(q_h^2) + eps)                  if q_unit      (no weight)
//   q_h <- q_h * (1 + coef * ln(floor((pos + 1) / every) + 1))           if every > 0
//   k_g <- k_g / sqrt(mean(k_g^2) + eps)                  if k_unit
//   v_g  = the k_g of the product, before its norm        if v_from_k    (the input then has no v columns)
//
// The output row is [q heads | k heads | v heads] in the compute dtype; k and v also go to the cache line
// (row = ring_rows ? pos % ring_rows : pos, page = page_table[seq, row / page_rows]; in a ring only tokens
// with pos >= len_after - ring_rows are written, as the rotary kernel does).
//
// One warp per (token, head slot); a lane holds elements lane, lane + 32, ... of the head.
#include "common.cuh"

TB_EXPORT_ERROR()

struct HeadNormKvArgs {
    const float* partial; int n_splits; long long split_stride, partial_row_stride;
    void* out; long long out_row_stride;      // [tokens][(n_heads + 2 n_kv_heads) * head_dim]
    int n_heads, n_kv_heads, head_dim;
    int q_unit, k_unit, v_from_k;
    float eps, temp_coef; int temp_every;
    const int* positions; const int* token_seq; const int* len_after;
    void* k_pool; void* v_pool; const int* page_table; int pt_stride; int page_rows; int ring_rows;
};

#define HN_MAX_PER_LANE 16        // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(256) headnorm_kv_kernel(HeadNormKvArgs a, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int in_slots = a.n_heads + a.n_kv_heads * (a.v_from_k ? 1 : 2);
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_tokens * in_slots) return;
    const int t = (int)(item / in_slots), hs = (int)(item % in_slots);
    const int hd = a.head_dim;
    const bool is_q = hs < a.n_heads;
    const bool is_k = !is_q && hs < a.n_heads + a.n_kv_heads;
    const int kvh = is_q ? 0 : (is_k ? hs - a.n_heads : hs - a.n_heads - a.n_kv_heads);
    const float* src = a.partial + (size_t)t * a.partial_row_stride + (size_t)hs * hd;
    const int pos = a.positions[t];

    float x[HN_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < HN_MAX_PER_LANE; k++) {
        const int i = lane + 32 * k;
        x[k] = 0.f;
        if (i < hd) {
            float v = src[i];
            for (int s = 1; s < a.n_splits; s++) v += src[(size_t)s * a.split_stride + i];
            x[k] = v;
            ss += v * v;
        }
    }
    float f = 1.f;
    if ((is_q && a.q_unit) || (is_k && a.k_unit)) {
        ss = warp_sum(ss);
        f = 1.0f / sqrtf(ss / (float)hd + a.eps);
    }
    if (is_q && a.temp_every > 0)
        f *= 1.0f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.0f);

    // where this token's k and v go in the cache (if anywhere)
    size_t cache_off = 0;
    bool store = false;
    if (!is_q && a.k_pool != nullptr) {
        const int b = a.token_seq[t];
        store = true;
        int r = pos;
        if (a.ring_rows > 0) { store = pos >= a.len_after[b] - a.ring_rows; r = pos % a.ring_rows; }
        if (store) {
            const int page = a.page_table[(size_t)b * a.pt_stride + r / a.page_rows];
            cache_off = (((size_t)page * a.n_kv_heads + kvh) * a.page_rows + (r % a.page_rows)) * hd;
        }
    }
    T* row = (T*)a.out + (size_t)t * a.out_row_stride;
    const int k_off = a.n_heads * hd, v_off = (a.n_heads + a.n_kv_heads) * hd;
    T* o_main = row + (is_q ? hs * hd : (is_k ? k_off + kvh * hd : v_off + kvh * hd));
    T* c_main = store ? (T*)(is_k ? a.k_pool : a.v_pool) + cache_off : nullptr;
    const bool also_v = is_k && a.v_from_k;
    T* o_v = also_v ? row + v_off + kvh * hd : nullptr;
    T* c_v = (also_v && store) ? (T*)a.v_pool + cache_off : nullptr;
#pragma unroll
    for (int k = 0; k < HN_MAX_PER_LANE; k++) {
        const int i = lane + 32 * k;
        if (i < hd) {
            const T y = from_f<T>(x[k] * f);
            o_main[i] = y;
            if (c_main) c_main[i] = y;
            if (also_v) {
                const T raw = from_f<T>(x[k]);
                o_v[i] = raw;
                if (c_v) c_v[i] = raw;
            }
        }
    }
}

extern "C" int tb_headnorm_kv(const HeadNormKvArgs* args, int out_dtype, int n_tokens, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    HeadNormKvArgs a = *args;
    if (a.head_dim <= 0 || a.head_dim > 32 * HN_MAX_PER_LANE)
        return tb_refuse("headnorm_kv: head_dim=%d (1..%d)", a.head_dim, 32 * HN_MAX_PER_LANE);
    if (a.n_heads <= 0 || a.n_kv_heads < 0) return tb_refuse("headnorm_kv: %d heads, %d kv heads", a.n_heads, a.n_kv_heads);
    if (a.partial == nullptr || a.n_splits < 1) return tb_refuse("headnorm_kv: needs the product's partial sums");
    if (a.k_pool != nullptr && (a.page_rows <= 0 || a.page_table == nullptr || a.v_pool == nullptr))
        return tb_refuse("headnorm_kv: a cache write needs page_rows > 0, a page table and both pools");
    if (a.ring_rows > 0 && a.ring_rows % a.page_rows != 0)
        return tb_refuse("headnorm_kv: ring_rows=%d must be a multiple of page_rows=%d", a.ring_rows, a.page_rows);
    const int in_slots = a.n_heads + a.n_kv_heads * (a.v_from_k ? 1 : 2);
    const long long items = (long long)n_tokens * in_slots;
    const long long blocks = (items + 7) / 8;
    if (blocks > 0x7fffffffLL) return tb_refuse("headnorm_kv: too many tokens");
    TB_DISPATCH_1(out_dtype, T, tb_launch(headnorm_kv_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, a, n_tokens));
    return tb_launch_status();
}
