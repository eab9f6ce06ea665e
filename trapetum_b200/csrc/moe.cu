// A feed-forward made of experts behind a router.
//
//   tb_moe_route     per token: logits z = R x (32-bit sums), scores s = sigmoid(z); choice scores s + correction;
//                    experts form `groups` equal groups of neighbours, a group's score is the sum of its
//                    `group_top` largest choice scores, experts outside the `keep` best groups cannot be chosen
//                    (their choice scores count as minus infinity); the `top` largest choice scores win (the
//                    lower index on a tie); weights are the winners' s divided by their sum + eps.  Also the
//                    shared expert's gate sigmoid(g . x), one number per token, if asked for.
//   tb_moe_gate_up   for every (token, chosen expert): act(G_e x) * (U_e x), act = silu
//   tb_moe_down      out[t] = sum_k weight[t,k] * D_e(t,k) a[t,k]  (+ gate[t] * shared[t], the shared expert's output
//                    given as 32-bit split-K partial sums), 32-bit
//
// The router is 32-bit throughout.  The experts' products take operands of the activations' dtype and sum in
// 32-bit; a[t,k] is rounded to the activations' dtype, the weighted sum over the experts is not.
#include "common.cuh"

TB_EXPORT_ERROR()

struct MoeRouteArgs {
    const void* x; long long x_stride;         // [T][W]
    const void* router;                        // [E][W]
    const float* correction;                   // [E] or null
    const void* shared_gate;                   // [W] or null
    int* idx; float* weight;                   // [T][top]
    float* gate;                               // [T] (if shared_gate)
    int n_tokens, W, E, top, groups, keep, group_top;
    float weight_eps;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_route_kernel(MoeRouteArgs a) {
    pdl_launch_dependents();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    float* score = smem + (size_t)warp * (2 * a.E + a.groups);
    float* choice = score + a.E;
    float* gscore = choice + a.E;
    pdl_wait();
    if (t >= a.n_tokens) return;
    const T* x = (const T*)a.x + (size_t)t * a.x_stride;
    for (int e = 0; e <= a.E; e++) {
        if (e == a.E && a.shared_gate == nullptr) break;
        const TW* w = (e < a.E) ? (const TW*)a.router + (size_t)e * a.W : (const TW*)a.shared_gate;
        float d = 0.f;
        for (int c = lane; c < a.W; c += 32) d = fmaf(to_f<T>(x[c]), to_f<TW>(w[c]), d);
        d = warp_sum(d);
        if (lane == 0) {
            const float s = 1.f / (1.f + expf(-d));
            if (e < a.E) { score[e] = s; choice[e] = s + (a.correction ? a.correction[e] : 0.f); }
            else a.gate[t] = s;
        }
    }
    __syncwarp();
    if (a.groups > 1) {
        const int per = a.E / a.groups;
        for (int g = lane; g < a.groups; g += 32) {
            int used[8];
            float sum = 0.f;
            for (int n = 0; n < a.group_top && n < per; n++) {
                float best = -INFINITY; int bi = -1;
                for (int j = 0; j < per; j++) {
                    bool taken = false;
                    for (int u = 0; u < n; u++) taken |= (used[u] == j);
                    if (!taken && (bi < 0 || choice[g * per + j] > best)) { best = choice[g * per + j]; bi = j; }
                }
                used[n] = bi; sum += best;
            }
            gscore[g] = sum;
        }
        __syncwarp();
        // the `keep` best groups stay; the others' experts cannot be chosen
        unsigned kept_lo = 0;                    // this lane's groups lane, lane+32, ... as bits
        for (int n = 0; n < a.keep; n++) {
            float v = -INFINITY; int i = 0x7fffffff;
            for (int g = lane; g < a.groups; g += 32)
                if (!((kept_lo >> (g >> 5)) & 1u) && (gscore[g] > v || i == 0x7fffffff)) { v = gscore[g]; i = g; }
            warp_argmax(v, i);
            if ((i & 31) == lane && i != 0x7fffffff) kept_lo |= 1u << (i >> 5);
        }
        for (int g = lane; g < a.groups; g += 32)
            if (!((kept_lo >> (g >> 5)) & 1u))
                for (int j = 0; j < per; j++) choice[g * per + j] = -INFINITY;
        __syncwarp();
    }
    float wsum = 0.f, mine = 0.f; int mine_i = 0;
    for (int n = 0; n < a.top; n++) {
        float v = -INFINITY; int i = 0x7fffffff;
        for (int e = lane; e < a.E; e += 32) if (choice[e] > v) { v = choice[e]; i = e; }
        warp_argmax(v, i);
        const float s = score[i];
        wsum += s;
        if (lane == (n & 31)) { mine = s; mine_i = i; if (n >= 32) { /* more than 32 winners: written below per round */ } }
        __syncwarp();
        if (lane == 0) choice[i] = -INFINITY;
        __syncwarp();
        if ((n & 31) == 31 || n == a.top - 1) {
            // park the round's winners; the weights are divided once the sum is known
            if (lane <= (n & 31)) { a.idx[(size_t)t * a.top + (n & ~31) + lane] = mine_i; a.weight[(size_t)t * a.top + (n & ~31) + lane] = mine; }
        }
    }
    __syncwarp();
    const float inv = 1.f / (wsum + a.weight_eps);
    for (int n = lane; n < a.top; n += 32) a.weight[(size_t)t * a.top + n] *= inv;
}

struct MoeExpertArgs {
    const void* x; long long x_stride;         // [T][W]
    const void* gate_w; const void* up_w;      // [E][ff][W]
    const void* down_w;                        // [E][W][ff]
    const int* idx; const float* weight;       // [T][top]
    void* act;                                 // [T * top][ff]
    const float* shared; int shared_splits; long long shared_split_stride;   // [splits][T][W] or null
    const float* gate;                         // [T] (with shared)
    float* out;                                // [T][W]
    int n_tokens, W, ff, top;
};

template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(MoeExpertArgs a) {
    pdl_launch_dependents();
    extern __shared__ float x_s[];              // [W]
    const int pair = blockIdx.x, t = pair / a.top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    pdl_wait();
    const int e = a.idx[pair];
    const T* x = (const T*)a.x + (size_t)t * a.x_stride;
    for (int c = threadIdx.x; c < a.W; c += blockDim.x) x_s[c] = to_f<T>(x[c]);
    __syncthreads();
    const T* gw = (const T*)a.gate_w + (size_t)e * a.ff * a.W;
    const T* uw = (const T*)a.up_w + (size_t)e * a.ff * a.W;
    for (int f = blockIdx.y * nwarp + warp; f < a.ff; f += gridDim.y * nwarp) {
        float g = 0.f, u = 0.f;
        for (int c = lane; c < a.W; c += 32) {
            g = fmaf(to_f<T>(gw[(size_t)f * a.W + c]), x_s[c], g);
            u = fmaf(to_f<T>(uw[(size_t)f * a.W + c]), x_s[c], u);
        }
        g = warp_sum(g); u = warp_sum(u);
        if (lane == 0) ((T*)a.act)[(size_t)pair * a.ff + f] = from_f<T>(g / (1.f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(MoeExpertArgs a) {
    pdl_launch_dependents();
    extern __shared__ float a_s[];              // [top][ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    pdl_wait();
    for (int i = threadIdx.x; i < a.top * a.ff; i += blockDim.x)
        a_s[i] = to_f<T>(((const T*)a.act)[(size_t)t * a.top * a.ff + i]) * a.weight[(size_t)t * a.top + i / a.ff];
    __syncthreads();
    for (int c = blockIdx.y * nwarp + warp; c < a.W; c += gridDim.y * nwarp) {
        float acc = 0.f;
        for (int k = 0; k < a.top; k++) {
            const T* dw = (const T*)a.down_w + ((size_t)a.idx[(size_t)t * a.top + k] * a.W + c) * a.ff;
            for (int f = lane; f < a.ff; f += 32) acc = fmaf(to_f<T>(dw[f]), a_s[k * a.ff + f], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (a.shared != nullptr) {
                float sh = 0.f;
                for (int s = 0; s < a.shared_splits; s++) sh += a.shared[(size_t)s * a.shared_split_stride + (size_t)t * a.W + c];
                acc = fmaf(a.gate[t], sh, acc);
            }
            a.out[(size_t)t * a.W + c] = acc;
        }
    }
}

extern "C" int tb_moe_route(const MoeRouteArgs* args, int x_dtype, int w_dtype, cudaStream_t stream) {
    const MoeRouteArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.E <= 0 || a.top < 1 || a.top > a.E || a.groups < 1 || a.E % a.groups || a.keep < 1 || a.keep > a.groups ||
        a.group_top < 1 || a.group_top > 8 || a.groups > 1024)
        return tb_refuse("moe_route: experts=%d top=%d groups=%d keep=%d group_top=%d", a.E, a.top, a.groups, a.keep, a.group_top);
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * a.E + a.groups) * sizeof(float);
    if (smem > 48 * 1024) return tb_refuse("moe_route: %d experts are more than one block holds", a.E);
    TB_DISPATCH_1(x_dtype, T, TB_DISPATCH_1(w_dtype, TW,
        tb_launch(moe_route_kernel<T, TW>, dim3((a.n_tokens + warps - 1) / warps), dim3(warps * 32), smem, stream, a)));
    return tb_launch_status();
}

extern "C" int tb_moe_gate_up(const MoeExpertArgs* args, int dtype, cudaStream_t stream) {
    const MoeExpertArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    if (a.W <= 0 || a.W > 12288 || a.ff <= 0 || a.top <= 0) return tb_refuse("moe: W=%d ff=%d top=%d", a.W, a.ff, a.top);
    const int ys = (a.ff + 63) / 64 < 32 ? (a.ff + 63) / 64 : 32;
    TB_DISPATCH_1(dtype, T, tb_launch(moe_gate_up_kernel<T>, dim3(a.n_tokens * a.top, ys), dim3(256), (size_t)a.W * sizeof(float), stream, a));
    return tb_launch_status();
}

extern "C" int tb_moe_down(const MoeExpertArgs* args, int dtype, cudaStream_t stream) {
    const MoeExpertArgs& a = *args;
    if (a.n_tokens <= 0) return 0;
    const size_t smem = (size_t)a.top * a.ff * sizeof(float);
    if (smem > 48 * 1024) return tb_refuse("moe_down: top=%d x ff=%d activations exceed one block's shared memory", a.top, a.ff);
    const int ys = (a.W + 63) / 64 < 32 ? (a.W + 63) / 64 : 32;
    TB_DISPATCH_1(dtype, T, tb_launch(moe_down_kernel<T>, dim3(a.n_tokens, ys), dim3(256), smem, stream, a));
    return tb_launch_status();
}
