#include "gemm.h"
#include "gemm_tc.h"
#include "kernels.h"
#include "../../include/vitb200.h"

#include <cstdlib>
#include <cstring>

namespace vitb200 {
namespace {

// Below this many multiply-adds a product is latency-bound either way and the
// exact FP32 kernel is used, which also keeps very small models (the host's
// own device test runs d_model = 32) at FP32 accuracy.
constexpr double kTensorCoreMinimumWork = 16.0 * 1024 * 1024;

int g_forced_precision = -1;

int default_precision() {
    if (g_forced_precision >= 0) {
        return g_forced_precision;
    }
    static int chosen = []() {
        const char *text = getenv("VITB200_GEMM");
        if (text && strcmp(text, "fp32") == 0) {
            return VITB200_PRECISION_FP32;
        }
        if (text && strcmp(text, "tf32") == 0) {
            return VITB200_PRECISION_TF32;
        }
        return VITB200_PRECISION_AUTO;
    }();
    return chosen;
}

// Decides whether `gemm` goes to the tensor cores: 1 yes, 0 no, -1 when the
// caller asked for TF32 explicitly and the layout cannot be served.  A TF32
// *default* (environment or vitb200_set_gemm_precision) means "wherever the
// layout allows" and falls back to FP32 quietly.
int use_tensor_cores(const TcGemm &gemm, int precision) {
    const bool explicit_request = precision != VITB200_PRECISION_AUTO;
    if (!explicit_request) {
        precision = default_precision();
    }
    if (precision == VITB200_PRECISION_FP32) {
        return 0;
    }
    const bool supported = gemm_tc_supported(gemm);
    if (precision == VITB200_PRECISION_TF32) {
        return supported ? 1 : (explicit_request ? -1 : 0);
    }
    const double work = double(gemm.m) * gemm.n * gemm.k;
    return supported && work >= kTensorCoreMinimumWork ? 1 : 0;
}

void simt(const TcGemm &g, cudaStream_t stream) {
    GemmOperands op;
    op.a = g.a;
    op.a_row = g.a_mn_major ? 1 : g.lda;
    op.a_col = g.a_mn_major ? g.lda : 1;
    op.b = g.b;
    op.b_row = g.b_mn_major ? g.ldb : 1;
    op.b_col = g.b_mn_major ? 1 : g.ldb;
    op.c = g.d;
    op.c_row = g.ldd;
    op.m = g.m;
    op.n = g.n;
    op.k = g.k;
    op.accumulate = g.accumulate ? 1 : 0;
    launch_gemm_simt(op, stream);
}

int run(const TcGemm &gemm, int precision, cudaStream_t stream) {
    const int tensor = use_tensor_cores(gemm, precision);
    if (tensor < 0) {
        return -1;
    }
    if (tensor == 1) {
        if (launch_gemm_tc(gemm, stream) == 0) {
            return 0;
        }
        if (precision == VITB200_PRECISION_TF32) {
            return -1;
        }
    }
    simt(gemm, stream);
    return 0;
}

}  // namespace

int gemm_default_precision() {
    return default_precision();
}

bool prefer_tensor_cores(int precision, double multiply_adds) {
    if (precision == VITB200_PRECISION_AUTO) {
        precision = default_precision();
    }
    if (precision == VITB200_PRECISION_FP32) {
        return false;
    }
    if (precision == VITB200_PRECISION_TF32) {
        return true;
    }
    return multiply_adds >= kTensorCoreMinimumWork;
}

extern unsigned long long g_fma_products;

void gemm_path_counters(unsigned long long *tensor_core,
                        unsigned long long *wide_tile, unsigned long long *fma) {
    *tensor_core = g_tc_products;
    *wide_tile = g_tc_wide_products;
    *fma = g_fma_products;
}

void gemm_set_default_precision(int precision) {
    g_forced_precision = precision;
}

int gemm_forward(const float *x, const float *w, float *y, int m, int k, int n,
                 int precision, cudaStream_t stream) {
    // Y[m,n] = X[m,k] W[k,n]: X has the reduction contiguous, W the output.
    TcGemm g = {x, w, y, nullptr, m, n, k, k, n, n, false, true, false};
    return run(g, precision, stream);
}

int gemm_forward_fused(const float *x, const float *w, float *y, int m, int k,
                       int n, const GemmEpilogue &e, int precision,
                       cudaStream_t stream) {
    TcGemm g = {x, w, y, e.bias, m, n, k, k, n, n, false, true, false};
    if (e.gelu_out) {
        g.d2 = e.gelu_out;
        g.ldd2 = n;
    } else if (e.residual_out) {
        g.d2 = e.residual_out;
        g.ldd2 = n;
        g.residual = e.residual;
        g.ld_residual = n;
    }
    const int tensor = use_tensor_cores(g, precision);
    if (tensor < 0) {
        return -1;
    }
    if (tensor == 1 && launch_gemm_tc(g, stream) == 0) {
        return 0;
    }
    if (tensor == 1 && precision == VITB200_PRECISION_TF32) {
        return -1;
    }
    // Separate kernels, same results.
    g.bias = nullptr;
    g.d2 = nullptr;
    g.residual = nullptr;
    simt(g, stream);
    const size_t count = size_t(m) * n;
    if (e.bias) {
        launch_bias_add(y, e.bias, y, m, n, stream);
    }
    if (e.gelu_out) {
        launch_gelu(y, e.gelu_out, count, stream);
    } else if (e.residual_out) {
        launch_add(e.residual, y, e.residual_out, count, stream);
    }
    return 0;
}

int gemm_backward_input(const float *w, const float *dy, float *dx, int m,
                        int k, int n, int precision, bool dx_add,
                        cudaStream_t stream) {
    // dX[m,k] += dY[m,n] W^T: both operands have the reduction (n) contiguous.
    TcGemm gx = {dy, w, dx, nullptr, m, k, n, n, n, k, false, false, dx_add};
    return run(gx, precision, stream);
}

int gemm_backward_weights(const float *x, const float *dy, float *dw, int m,
                          int k, int n, int precision, cudaStream_t stream) {
    // dW[k,n] += X^T dY: both operands have their output index contiguous.
    TcGemm gw = {x, dy, dw, nullptr, k, n, m, k, n, n, true, true, true};
    return run(gw, precision, stream);
}

int gemm_backward(const float *x, const float *w, const float *dy, float *dx,
                  float *dw, int m, int k, int n, int precision, bool dx_add,
                  cudaStream_t stream) {
    if (gemm_backward_input(w, dy, dx, m, k, n, precision, dx_add, stream) != 0) {
        return -1;
    }
    return gemm_backward_weights(x, dy, dw, m, k, n, precision, stream);
}

bool gemm_backward_input_gelu_supported(const float *w, const float *dy,
                                        const float *gelu_input,
                                        float *d_gelu_input, int m, int k,
                                        int n, int precision) {
    TcGemm g = {dy, w, d_gelu_input, nullptr, m, k, n, n, n, k, false, false, false};
    g.gelu_input = gelu_input;
    g.ld_gelu_input = k;
    return use_tensor_cores(g, precision) == 1;
}

int gemm_backward_input_gelu(const float *w, const float *dy,
                             const float *gelu_input, float *d_gelu_input,
                             float *column_partials, int m, int k, int n,
                             int precision, cudaStream_t stream) {
    TcGemm g = {dy, w, d_gelu_input, nullptr, m, k, n, n, n, k, false, false, false};
    g.gelu_input = gelu_input;
    g.ld_gelu_input = k;
    g.column_partials = column_partials;
    if (use_tensor_cores(g, precision) != 1) {
        return -1;
    }
    return launch_gemm_tc(g, stream);
}

}  // namespace vitb200
