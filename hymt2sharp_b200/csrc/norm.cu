// Row-wise RMSNorm: y = x * (1 / sqrt(sum(x^2)/dim + eps)) * gain, all in float32
// (src/HyMT2Sharp/Ops.cs:29-89; scale at :62, product order at :69-72).
// `rows_index`, when given, picks the input rows (y[r] = norm(x[rows_index[r]])):
// the final norm runs only on the rows whose logits are wanted.
#include "common.cuh"

template <typename TX, typename TW, typename TY>
__global__ void rmsnorm_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ gain,
                               const int* __restrict__ rows_index, int dim, float eps) {
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
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        dst[i] = from_float<TY>(to_float(src[i]) * scale * to_float(gain[i]));
}

HYMT2_API int hymt2_rmsnorm(void* y, int y_dtype, const void* x, int x_dtype, const void* gain, int gain_dtype,
                            const int* rows_index, int rows, int dim, float eps, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", rows, dim);
    const int threads = dim >= 1024 ? 256 : (dim >= 256 ? 128 : 32);
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(y_dtype, TY,
        (launch_pdl(rmsnorm_kernel<TX, TW, TY>, dim3(rows), dim3(threads), 0, stream, (TY*)y, (const TX*)x,
                    (const TW*)gain, rows_index, dim, eps)))));
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
