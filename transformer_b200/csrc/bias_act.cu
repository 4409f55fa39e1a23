// Biases of a feed-forward whose projections have them, applied to the products' results.
//
//   h[t, c] = silu(gu[t, c] + b[c]) * (gu[t, di + c] + b[di + c])        the (gate, up) pair with its biases
//   y[t, c] += b[c]                                                       the down projection's
// Biases are float; the sums and the activation are float, one rounding at the store.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256) bias_glu_kernel(const T* __restrict__ gu, const float* __restrict__ bias,
                                                       T* __restrict__ h, long long n, int di) {
    pdl_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / di;
        const int c = (int)(i - t * di);
        const float g = ldf(gu + t * 2 * di + c) + bias[c];
        const float u = ldf(gu + t * 2 * di + di + c) + bias[di + c];
        stf(h + i, g / (1.0f + expf(-g)) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) add_bias_kernel(T* __restrict__ y, const float* __restrict__ bias, long long n, int d) {
    pdl_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        stf(y + i, ldf(y + i) + bias[i % d]);
}

static int grid_for(long long n) {
    const long long blocks = (n + 255) / 256;
    return (int)(blocks > 8192 ? 8192 : blocks);
}

extern "C" {
#define TB_BIAS(SFX, T)                                                                                               \
    int tb_bias_glu_##SFX(const void* gu, const float* bias, void* h, int nt, int di, cudaStream_t s) {               \
        if (nt < 0 || di <= 0 || !bias) return TB_ERR_ARG;                                                            \
        if (nt == 0) return 0;                                                                                        \
        const long long n = (long long)nt * di;                                                                       \
        TB_LAUNCH((bias_glu_kernel<T>), grid_for(n), 256, 0, s, (const T*)gu, bias, (T*)h, n, di);                    \
        return tb_last_error();                                                                                       \
    }                                                                                                                 \
    int tb_add_bias_##SFX(void* y, const float* bias, int nt, int d, cudaStream_t s) {                                \
        if (nt < 0 || d <= 0 || !bias) return TB_ERR_ARG;                                                             \
        if (nt == 0) return 0;                                                                                        \
        const long long n = (long long)nt * d;                                                                        \
        TB_LAUNCH((add_bias_kernel<T>), grid_for(n), 256, 0, s, (T*)y, bias, n, d);                                   \
        return tb_last_error();                                                                                       \
    }
TB_BIAS(f32, float)
TB_BIAS(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_bias_glu_f32)
TB_TAPE_REGISTER(tb_bias_glu_bf16)
TB_TAPE_REGISTER(tb_add_bias_f32)
TB_TAPE_REGISTER(tb_add_bias_bf16)
