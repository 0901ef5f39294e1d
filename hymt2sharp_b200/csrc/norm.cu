// Row-wise RMSNorm: y = x * (1 / sqrt(sum(x^2)/dim + eps)) * gain, all in float32
// (src/HyMT2Sharp/Ops.cs:29-89; scale at :62, product order at :69-72).  `out_scale` multiplies the
// result (1 for this architecture; a model that scales its logits gives the factor to its final norm).
// `rows_index`, when given, picks the input rows (y[r] = norm(x[rows_index[r]])):
// the final norm runs only on the rows whose logits are wanted.
#include "common.cuh"

template <typename TX, typename TW, typename TY>
__global__ void rmsnorm_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ gain,
                               const int* __restrict__ rows_index, int dim, float eps, float out_scale) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const TX* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = to_float(src[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    TY* dst = y + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = to_float(src[i]) * scale * to_float(gain[i]);
        dst[i] = from_float<TY>(out_scale == 1.0f ? v : v * out_scale);
    }
}

// The common case in one pass: float32 rows whose 8 values per thread stay in registers between
// the sum of squares and the scaling; 16-byte loads, one 16-byte store of 8 bfloat16 per thread.
template <typename TW>
__global__ void rmsnorm_f32_bf16_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ x,
                                        const TW* __restrict__ gain, const int* __restrict__ rows_index, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim;
    const int c = threadIdx.x * 8;
    float v[8];
    const float4 a = *reinterpret_cast<const float4*>(src + c), b = *reinterpret_cast<const float4*>(src + c + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
        h[i] = __floats2bfloat162_rn(v[2 * i] * scale * to_float(gain[c + 2 * i]), v[2 * i + 1] * scale * to_float(gain[c + 2 * i + 1]));
    *reinterpret_cast<uint4*>(y + (size_t)r * dim + c) = *reinterpret_cast<uint4*>(h);
}

HYMT2_API int hymt2_rmsnorm(void* y, int y_dtype, const void* x, int x_dtype, const void* gain, int gain_dtype,
                            const int* rows_index, int rows, int dim, float eps, float out_scale, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", rows, dim);
    if (out_scale == 1.0f && x_dtype == HYMT2_F32 && y_dtype == HYMT2_BF16 && dim % 256 == 0 && dim <= 8192 &&
        (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
        cudaError_t e;
        if (gain_dtype == HYMT2_BF16)
            e = launch_pdl(rmsnorm_f32_bf16_kernel<__nv_bfloat16>, dim3(rows), dim3(dim / 8), 0, stream, (__nv_bfloat16*)y,
                           (const float*)x, (const __nv_bfloat16*)gain, rows_index, dim, eps);
        else
            e = launch_pdl(rmsnorm_f32_bf16_kernel<float>, dim3(rows), dim3(dim / 8), 0, stream, (__nv_bfloat16*)y,
                           (const float*)x, (const float*)gain, rows_index, dim, eps);
        (void)e;
        return hymt2_check_launch("rmsnorm");
    }
    const int threads = dim >= 1024 ? 256 : (dim >= 256 ? 128 : 32);
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(y_dtype, TY,
        (launch_pdl(rmsnorm_kernel<TX, TW, TY>, dim3(rows), dim3(threads), 0, stream, (TY*)y, (const TX*)x,
                    (const TW*)gain, rows_index, dim, eps, out_scale)))));
    return hymt2_check_launch("rmsnorm");
}

// a = gate / (1 + exp(-gate)) * up on a [rows, 2*width] input whose first half of every row is
// the gate and whose second half is the up projection (src/HyMT2Sharp/Ops.cs:999-1055).
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int width, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t r = i / width;
    int c = (int)(i - r * width);
    float g = to_float(gate_up[r * 2 * width + c]);
    float u = to_float(gate_up[r * 2 * width + width + c]);
    out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

HYMT2_API int hymt2_silu_mul(void* out, const void* gate_up, int dtype, int rows, int width, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && width > 0, "silu_mul: bad sizes rows=%d width=%d", rows, width);
    size_t total = (size_t)rows * width;
    unsigned blocks = (unsigned)((total + 255) / 256);
    HYMT2_DISPATCH_DTYPE(dtype, T, silu_mul_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, (const T*)gate_up, width, total));
    return hymt2_check_launch("silu_mul");
}
