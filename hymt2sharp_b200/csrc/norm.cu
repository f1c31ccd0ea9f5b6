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

// RMSNorm in groups: a row is cut into `groups` equal consecutive parts, each part is divided by its own
// sqrt(mean(part^2) + eps), and the whole is multiplied by the gain; all in float32.  One block per (row, part).
// `ADD`: the result is added to y (float32 rows that already hold something: a residual stream that takes a
// sublayer's output after a norm) instead of stored.
template <typename TX, typename TW, typename TY, bool ADD>
__global__ void rmsnorm_groups_kernel(TY* __restrict__ y, const TX* __restrict__ x, const TW* __restrict__ gain,
                                      const int* __restrict__ rows_index, int dim, int part, float eps, float out_scale) {
    __shared__ float scratch[33];
    pdl_wait();   // everything in front is complete before anything is read; then the next kernel may be set up meanwhile
    pdl_launch_dependents();
    const int r = blockIdx.x, g = blockIdx.y;
    const TX* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim + (size_t)g * part;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = to_float(src[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)part + eps);
    TY* dst = y + (size_t)r * dim + (size_t)g * part;
    const TW* gn = gain + (size_t)g * part;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        float v = to_float(src[i]) * scale * to_float(gn[i]);
        if (out_scale != 1.0f) v *= out_scale;
        if constexpr (ADD) dst[i] = from_float<TY>(to_float(dst[i]) + v);
        else dst[i] = from_float<TY>(v);
    }
}

// The same for float32 rows whose parts are whole pieces of four values: 16-byte loads, and 16- or 8-byte stores.
template <typename TW, typename TY, bool ADD>
__global__ void rmsnorm_groups_vec_kernel(TY* __restrict__ y, const float* __restrict__ x, const TW* __restrict__ gain,
                                          const int* __restrict__ rows_index, int dim, int part, float eps, float out_scale) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, g = blockIdx.y;
    const float* src = x + (size_t)(rows_index ? rows_index[r] : r) * dim + (size_t)g * part;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = block_sum(ss, scratch);
    const float scale = out_scale / sqrtf(ss / (float)part + eps);
    TY* dst = y + (size_t)r * dim + (size_t)g * part;
    const TW* gn = gain + (size_t)g * part;
    for (int i = threadIdx.x * 4; i < part; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        float o[4] = {v.x * scale * to_float(gn[i]), v.y * scale * to_float(gn[i + 1]), v.z * scale * to_float(gn[i + 2]),
                      v.w * scale * to_float(gn[i + 3])};
        if constexpr (sizeof(TY) == 4) {
            float4* d4 = reinterpret_cast<float4*>(dst + i);
            if constexpr (ADD) {
                const float4 old = *d4;
                o[0] += old.x; o[1] += old.y; o[2] += old.z; o[3] += old.w;
            }
            *d4 = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(dst + i) = *reinterpret_cast<const uint2*>(h);
        }
    }
}

// Two norms around the residual sum in one pass over a row part: y (float32) += norm_a(x), then h = norm_b(y) of the new y
// (gain_b null: h = the new y itself, rounded to h's type).
// (A sublayer's output joins the residual through a norm, and the next sublayer reads the residual through another.)
// A thread meets the same entries in every loop, so only the two sums of squares cross threads.
template <typename TW, typename TH>
__global__ void rmsnorm_groups_add_norm_kernel(float* __restrict__ y, const float* __restrict__ x, const TW* __restrict__ gain_a,
                                               TH* __restrict__ h, const TW* __restrict__ gain_b, int dim, int part, float eps_a,
                                               float eps_b) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, g = blockIdx.y;
    const size_t off = (size_t)r * dim + (size_t)g * part;
    const float* src = x + off;
    float* res = y + off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, scratch);
    const float scale_a = 1.0f / sqrtf(ss / (float)part + eps_a);
    const TW* ga = gain_a + (size_t)g * part;
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = res[i] + src[i] * scale_a * to_float(ga[i]);
        res[i] = v;
        ss2 = fmaf(v, v, ss2);
    }
    TH* dst = h + off;
    if (gain_b == nullptr) {   // no second norm: the next sublayer reads the new rows as they are, in its own type
        for (int i = threadIdx.x; i < part; i += blockDim.x) dst[i] = from_float<TH>(res[i]);
        return;
    }
    ss2 = block_sum(ss2, scratch);
    const float scale_b = 1.0f / sqrtf(ss2 / (float)part + eps_b);
    const TW* gb = gain_b + (size_t)g * part;
    for (int i = threadIdx.x; i < part; i += blockDim.x) dst[i] = from_float<TH>(res[i] * scale_b * to_float(gb[i]));
}

HYMT2_API int hymt2_rmsnorm_groups_add_norm(float* y, const float* x, const void* gain_a, void* h, int h_dtype, const void* gain_b,
                                            int gain_dtype, int rows, int dim, int groups, float eps_a, float eps_b,
                                            cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0 && groups > 0 && dim % groups == 0 && groups <= 65535,
                  "rmsnorm: bad sizes rows=%d dim=%d groups=%d", rows, dim, groups);
    const int part = dim / groups;
    const int threads = part >= 1024 ? 256 : (part >= 256 ? 128 : (part >= 64 ? 64 : 32));
    const dim3 grid(rows, groups);
    HYMT2_DISPATCH_DTYPE(gain_dtype, TW, HYMT2_DISPATCH_DTYPE(h_dtype, TH,
        (launch_pdl(rmsnorm_groups_add_norm_kernel<TW, TH>, grid, dim3(threads), 0, stream, y, x, (const TW*)gain_a, (TH*)h,
                    (const TW*)gain_b, dim, part, eps_a, eps_b))));
    return hymt2_check_launch("rmsnorm_groups_add_norm");
}

HYMT2_API int hymt2_rmsnorm_groups(void* y, int y_dtype, const void* x, int x_dtype, const void* gain, int gain_dtype,
                                   const int* rows_index, int rows, int dim, int groups, float eps, float out_scale,
                                   int add, cudaStream_t stream) {
    if (rows == 0) return HYMT2_OK;
    HYMT2_REQUIRE(rows > 0 && dim > 0 && groups > 0 && dim % groups == 0 && groups <= 65535,
                  "rmsnorm: bad sizes rows=%d dim=%d groups=%d", rows, dim, groups);
    HYMT2_REQUIRE(!add || y_dtype == HYMT2_F32, "rmsnorm: adding into the output needs float32 rows");
    const int part = dim / groups;
    const int threads = part >= 1024 ? 256 : (part >= 256 ? 128 : (part >= 64 ? 64 : 32));
    const dim3 grid(rows, groups);
    if (x_dtype == HYMT2_F32 && part % 4 == 0 && dim % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
        const int vt = part >= 1024 ? 256 : (part >= 512 ? 128 : (part >= 256 ? 64 : 32));
        HYMT2_DISPATCH_DTYPE(gain_dtype, TW, {
            if (add)
                launch_pdl(rmsnorm_groups_vec_kernel<TW, float, true>, grid, dim3(vt), 0, stream, (float*)y, (const float*)x, (const TW*)gain,
                           rows_index, dim, part, eps, out_scale);
            else
                HYMT2_DISPATCH_DTYPE(y_dtype, TY, (launch_pdl(rmsnorm_groups_vec_kernel<TW, TY, false>, grid, dim3(vt), 0, stream, (TY*)y,
                                                              (const float*)x, (const TW*)gain, rows_index, dim, part, eps, out_scale)));
        });
        return hymt2_check_launch("rmsnorm_groups");
    }
    HYMT2_DISPATCH_DTYPE(x_dtype, TX, HYMT2_DISPATCH_DTYPE(gain_dtype, TW, {
        if (add) {
            launch_pdl(rmsnorm_groups_kernel<TX, TW, float, true>, grid, dim3(threads), 0, stream, (float*)y, (const TX*)x, (const TW*)gain,
                       rows_index, dim, part, eps, out_scale);
        } else {
            HYMT2_DISPATCH_DTYPE(y_dtype, TY, (launch_pdl(rmsnorm_groups_kernel<TX, TW, TY, false>, grid, dim3(threads), 0, stream,
                (TY*)y, (const TX*)x, (const TW*)gain, rows_index, dim, part, eps, out_scale)));
        }
    }));
    return hymt2_check_launch("rmsnorm_groups");
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
