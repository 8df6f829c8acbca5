// fp32 contraction with the summation order of the reference's mat_dot_t
// (mat_express_t.hpp:730-736): each output element is s = 0; s += a(i,k) * b(k,j)
// for k ascending, multiply and add rounded separately.  Used for the
// reference-exact fp32 paths (small models, parity tests); the bf16 projections of
// the large model go through the tcgen05 kernel instead.
#include "common.cuh"

namespace jsm {

struct MatD {
    const float* p;
    int rows, cols;
    long long rs, cs;
};

constexpr int TM = 64, TN = 64, TK = 16;

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }

__global__ void __launch_bounds__(256) dot_f32_kernel(MatD A, MatD B, MatD bias, int has_bias, int epilogue, MatD R,
                                                      float* Cp, long long crs, long long ccs, int M, int N, int K) {
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // A tile: TM x TK, B tile: TK x TN (1024 elements each, 4 per thread)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int idx = threadIdx.x + e * 256;
            // choose the faster-varying index along the contiguous axis of each operand
            int am, ak;
            if (A.cs == 1) { ak = idx % TK; am = idx / TK; } else { am = idx % TM; ak = idx / TM; }
            int gm = m0 + am, gk = k0 + ak;
            As[ak][am] = (gm < M && gk < K) ? A.p[gm * A.rs + gk * A.cs] : 0.0f;
            int bk, bn;
            if (B.cs == 1) { bn = idx % TN; bk = idx / TN; } else { bk = idx % TK; bn = idx / TK; }
            int gn = n0 + bn;
            gk = k0 + bk;
            Bs[bk][bn] = (gn < N && gk < K) ? B.p[gk * B.rs + gn * B.cs] : 0.0f;
        }
        __syncthreads();
        const int kmax = (K - k0) < TK ? (K - k0) : TK;  // never add the zero padding: -0.0 + 0.0 would flip a sign
        for (int k = 0; k < kmax; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float v = acc[i][j];
                if (has_bias) v = __fadd_rn(v, bias.p[(m % bias.rows) * bias.rs + (n % bias.cols) * bias.cs]);
                if (epilogue == 1) v = v > 0.0f ? v : 0.0f * v;
                else if (epilogue == 2) v = gelu_f(v);
                else if (epilogue == 3) v = __fadd_rn(v, R.p[(m % R.rows) * R.rs + (n % R.cols) * R.cs]);
                Cp[m * crs + n * ccs] = v;
            }
        }
}

static MatD to_d(const jsm_mat& m) {
    MatD d;
    d.p = reinterpret_cast<const float*>(m.data);
    d.rows = m.rows; d.cols = m.cols; d.rs = m.row_stride; d.cs = m.col_stride;
    return d;
}

}  // namespace jsm

using namespace jsm;

extern "C" jsm_status jsm_dot_f32(jsm_mat A, jsm_mat B, const jsm_mat* bias, int epilogue, const jsm_mat* R, jsm_mat Cm,
                                  void* stream) {
    if (A.cols != B.rows)
        JSM_FAIL(JSM_INVALID_ARG, "mat_dot_t: inner dimensions do not match for dot product (%d x %d . %d x %d)", A.rows,
                 A.cols, B.rows, B.cols);
    if (A.dtype != JSM_F32 || B.dtype != JSM_F32 || Cm.dtype != JSM_F32) JSM_FAIL(JSM_UNSUPPORTED, "jsm_dot_f32: f32 only");
    if (Cm.rows != A.rows || Cm.cols != B.cols)
        JSM_FAIL(JSM_SHAPE, "jsm_dot_f32: output is %d x %d, product is %d x %d", Cm.rows, Cm.cols, A.rows, B.cols);
    if (epilogue < 0 || epilogue > 3 || (epilogue == 3 && !R)) JSM_FAIL(JSM_INVALID_ARG, "jsm_dot_f32: epilogue %d", epilogue);
    if (A.rows == 0 || B.cols == 0) return JSM_OK;
    if (!A.data || !B.data || !Cm.data) JSM_FAIL(JSM_INVALID_ARG, "jsm_dot_f32: null operand");
    if ((bias && (bias->dtype != JSM_F32 || !bias->data || bias->rows <= 0 || bias->cols <= 0)) ||
        (R && (R->dtype != JSM_F32 || !R->data || R->rows <= 0 || R->cols <= 0)))
        JSM_FAIL(JSM_INVALID_ARG, "jsm_dot_f32: bad bias / residual operand");
    MatD bd = bias ? to_d(*bias) : MatD{nullptr, 1, 1, 0, 0};
    MatD rd = R ? to_d(*R) : MatD{nullptr, 1, 1, 0, 0};
    dim3 grid((Cm.cols + TN - 1) / TN, (Cm.rows + TM - 1) / TM);
    dot_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(to_d(A), to_d(B), bd, bias ? 1 : 0, epilogue, rd,
                                                        reinterpret_cast<float*>(Cm.data), Cm.row_stride, Cm.col_stride,
                                                        A.rows, B.cols, A.cols);
    JSM_LAUNCH_CHECK();
    return JSM_OK;
}
