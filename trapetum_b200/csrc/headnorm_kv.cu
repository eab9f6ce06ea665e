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
// One warp per (token, head slot); a lane holds groups of four neighbouring elements of the head (single elements
// when a size or an address does not allow 16-byte accesses).
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

template <typename T> __device__ __forceinline__ void store4(T* p, const float* f);
template <> __device__ __forceinline__ void store4<float>(float* p, const float* f) { *(float4*)p = make_float4(f[0], f[1], f[2], f[3]); }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const float* f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    *(uint2*)p = make_uint2(*(uint32_t*)&a, *(uint32_t*)&b);
}

// VEC = 4: head_dim and all row strides are multiples of 4 and the bases 16-byte aligned; a lane then holds groups of
// four neighbouring elements (one 16-byte load per split, one 8- or 16-byte store per destination).
// AT_ONCE: head slots a warp works on at a time (their loads are requested together): four for many tokens, one for
// few, where a warp's chain of dependent loads (position, page, rows) is the launch's whole time.

// GROUPS: groups of VEC elements a lane holds of one head (head_dim <= 32 * VEC * GROUPS).
template <typename T, int VEC, int GROUPS, int AT_ONCE>
__global__ void __launch_bounds__(256) headnorm_kv_kernel(HeadNormKvArgs a, int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int in_slots = a.n_heads + a.n_kv_heads * (a.v_from_k ? 1 : 2);
    const int n_items = n_tokens * in_slots;                         // (the host refuses what does not fit 31 bits)
    const int item0 = (blockIdx.x * (blockDim.x >> 5) + warp) * AT_ONCE;
    if (item0 >= n_items) return;
    const int hd = a.head_dim;
    constexpr int groups = GROUPS;

    float x[AT_ONCE][GROUPS][VEC];
#pragma unroll
    for (int u = 0; u < AT_ONCE; u++) {
        const int item = item0 + u;
        const int t = item / in_slots, hs = item - t * in_slots;
        const float* src = a.partial + (size_t)t * a.partial_row_stride + (size_t)hs * hd;
#pragma unroll
        for (int k = 0; k < GROUPS; k++) {
            const int i = (lane + 32 * k) * VEC;
#pragma unroll
            for (int e = 0; e < VEC; e++) x[u][k][e] = 0.f;
            if (item < n_items && k < groups && i < hd) {
                for (int s = 0; s < a.n_splits; s++) {               // added in split order
                    const float* q = src + (size_t)s * a.split_stride + i;
                    if (VEC == 4) {
                        const float4 v = *(const float4*)q;
                        x[u][k][0] += v.x; x[u][k][1] += v.y; x[u][k][2] += v.z; x[u][k][3] += v.w;
                    } else {
                        x[u][k][0] += q[0];
                    }
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < AT_ONCE; u++) {
        const int item = item0 + u;
        if (item >= n_items) break;                                  // (the same in every lane)
        const int t = item / in_slots, hs = item - t * in_slots;
        const bool is_q = hs < a.n_heads;
        const bool is_k = !is_q && hs < a.n_heads + a.n_kv_heads;
        const int kvh = is_q ? 0 : (is_k ? hs - a.n_heads : hs - a.n_heads - a.n_kv_heads);
        const int pos = a.positions[t];
        float f = 1.f;
        if ((is_q && a.q_unit) || (is_k && a.k_unit)) {
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < GROUPS; k++)
#pragma unroll
                for (int e = 0; e < VEC; e++) ss += x[u][k][e] * x[u][k][e];
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
        for (int k = 0; k < GROUPS; k++) {
            const int i = (lane + 32 * k) * VEC;
            if (k < groups && i < hd) {
                float y[VEC];
#pragma unroll
                for (int e = 0; e < VEC; e++) y[e] = x[u][k][e] * f;
                if (VEC == 4) {
                    store4<T>(o_main + i, y);
                    if (c_main) store4<T>(c_main + i, y);
                    if (also_v) { store4<T>(o_v + i, x[u][k]); if (c_v) store4<T>(c_v + i, x[u][k]); }
                } else {
                    const T yy = from_f<T>(y[0]);
                    o_main[i] = yy;
                    if (c_main) c_main[i] = yy;
                    if (also_v) { const T raw = from_f<T>(x[u][k][0]); o_v[i] = raw; if (c_v) c_v[i] = raw; }
                }
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
    const int at_once = items >= 8192 ? 4 : 1;
    const long long blocks = (items + 8 * at_once - 1) / (8 * at_once);
    if (items + 32 > 0x7fffffffLL) return tb_refuse("headnorm_kv: too many tokens");
    auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = a.head_dim % 4 == 0 && a.split_stride % 4 == 0 && a.partial_row_stride % 4 == 0 &&
                     a.out_row_stride % 4 == 0 && al16(a.partial) && al16(a.out) && al16(a.k_pool) && al16(a.v_pool);
#define HN(VEC_, G_) do { \
        if (at_once == 4) TB_DISPATCH_1(out_dtype, T, tb_launch(headnorm_kv_kernel<T, VEC_, G_, 4>, dim3((unsigned)blocks), dim3(256), 0, stream, a, n_tokens)); \
        else TB_DISPATCH_1(out_dtype, T, tb_launch(headnorm_kv_kernel<T, VEC_, G_, 1>, dim3((unsigned)blocks), dim3(256), 0, stream, a, n_tokens)); \
    } while (0)
    if (vec) { if (a.head_dim <= 128) HN(4, 1); else if (a.head_dim <= 256) HN(4, 2); else HN(4, 4); }
    else { if (a.head_dim <= 128) HN(1, 4); else HN(1, 16); }
#undef HN
    return tb_launch_status();
}
