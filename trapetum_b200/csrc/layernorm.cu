// Layer norm with weight and bias, fused with the residual sum that precedes it, and the row-wise
// additions to the residual stream.
//
//   tb_add_layernorm   h += a (if a is given: a branch output [rows, width] in 32 or 16 bits, or 32-bit
//                      split-K partial sums [splits, rows, width], added in split order);
//                      y = (h - mean) / sqrt(var + eps) * w + b
//   tb_add_rows        h += rows + vector   (either may be absent)
//
// Everything is 32-bit: the sum, the mean, the variance (mean of the squared deviations from the
// mean, taken in a second pass over the row, which the CTA keeps in shared memory), scale and shift.
// Only y is rounded to the output dtype.  One CTA per row.
#include "common.cuh"

TB_EXPORT_ERROR()

template <typename TA, typename TO>
__global__ void __launch_bounds__(256) add_layernorm_kernel(float* __restrict__ h, const TA* __restrict__ a, int n_splits,
                                                            long long split_stride, const float* __restrict__ w,
                                                            const float* __restrict__ b, float eps, TO* __restrict__ y,
                                                            int width) {
    pdl_launch_dependents();
    extern __shared__ float row_s[];
    __shared__ float red[33];
    const size_t row = blockIdx.x;
    pdl_wait();
    float* hr = h + row * width;
    float sum = 0.f;
    const bool vec = (width & 3) == 0 && sizeof(TA) == 4;           // 16-byte pieces: rows of 32-bit numbers, width a multiple of 4
    if (vec) {
        for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
            float4 v = *(const float4*)(hr + c);
            if (a != nullptr) {
                for (int s = 0; s < n_splits; s++) {
                    const float4 u = *(const float4*)((const float*)a + (size_t)s * split_stride + row * width + c);
                    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
                }
                *(float4*)(hr + c) = v;
            }
            *(float4*)(row_s + c) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float v = hr[c];
            if (a != nullptr) {
                for (int s = 0; s < n_splits; s++) v += to_f<TA>(a[(size_t)s * split_stride + row * width + c]);
                hr[c] = v;
            }
            row_s[c] = v;
            sum += v;
        }
    }
    const float mean = block_sum(sum, red) / (float)width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) { const float d = row_s[c] - mean; sq = fmaf(d, d, sq); }
    const float rstd = 1.f / sqrtf(block_sum(sq, red) / (float)width + eps);
    TO* yr = y + row * width;
    if ((width & 3) == 0) {
        for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
            const float4 v = *(const float4*)(row_s + c), ww = *(const float4*)(w + c), bb = *(const float4*)(b + c);
            const float o0 = (v.x - mean) * rstd * ww.x + bb.x, o1 = (v.y - mean) * rstd * ww.y + bb.y;
            const float o2 = (v.z - mean) * rstd * ww.z + bb.z, o3 = (v.w - mean) * rstd * ww.w + bb.w;
            if (sizeof(TO) == 4) *(float4*)((float*)yr + c) = make_float4(o0, o1, o2, o3);
            else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
                *(uint2*)((bf16*)yr + c) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
            }
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) yr[c] = from_f<TO>((row_s[c] - mean) * rstd * w[c] + b[c]);
    }
}

__global__ void add_rows_kernel(float* __restrict__ h, const float* __restrict__ rows, const float* __restrict__ vec,
                                long long n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = h[i];
    if (rows != nullptr) v += rows[i];
    if (vec != nullptr) v += vec[i % width];
    h[i] = v;
}

extern "C" int tb_add_layernorm(float* h, const void* a, int a_dtype, int n_splits, long long split_stride, const float* w,
                                const float* b, float eps, void* y, int y_dtype, int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || width > 48 * 1024 / 4) return tb_refuse("layernorm: width %d is outside [1, 12288]", width);
    if (a != nullptr && n_splits > 1 && a_dtype != TB_F32) return tb_refuse("layernorm: partial sums must be 32-bit");
    if (a == nullptr) n_splits = 0;
    const size_t smem = (size_t)width * sizeof(float);
    TB_DISPATCH_1(a_dtype, TA, TB_DISPATCH_1(y_dtype, TO,
        tb_launch(add_layernorm_kernel<TA, TO>, dim3(rows), dim3(256), smem, stream, h, (const TA*)a, n_splits, split_stride,
                  w, b, eps, (TO*)y, width)));
    return tb_launch_status();
}

extern "C" int tb_add_rows(float* h, const float* rows, const float* vec, int n_rows, int width, cudaStream_t stream) {
    const long long n = (long long)n_rows * width;
    if (n <= 0) return 0;
    tb_launch(add_rows_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, h, rows, vec, n, width);
    return tb_launch_status();
}
