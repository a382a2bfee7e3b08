// THNN_Cuda* entry points: the reference's C ABI for the convolutional hot path, over a minimal
// THC-compatible tensor struct.  Each wrapper does what the reference's host wrapper does around its
// kernels — shape checks with the same messages, resizing outputs in place, contiguous copies of
// strided inputs — and then calls the flat C ABI (cunn_b200.h) on the state's current stream.
// Errors go through the state's error hook (TH's THError); if the hook returns, the entry point returns.
#include "common.cuh"
#include "../../include/THCUNN_b200.h"   // with CUNN_B200_USE_REAL_THC this pulls in cutorch's <THC/THC.h>

#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>

// Tensor and state access goes through one of two back-ends with the same helper names:
//   thc_backend_builtin.inc  the library's own state and tensor struct (default; what the tests drive);
//   thc_backend_real.inc     cutorch's libTHC (THCState_getCurrentStream, THCudaTensor_newContiguous,
//                            THCudaTensor_resizeNd, THError ...), for a build inside a Lua-Torch install.
#ifdef CUNN_B200_USE_REAL_THC
#include "thc_backend_real.inc"
#else
#include "thc_backend_builtin.inc"
#endif

extern "C" void thcunn_b200_not_implemented(THCState *state, const char *name)
{
    if (state) raise(state, "%s is not implemented in this build (only the convolutional hot path is)", name);
    else fprintf(stderr, "THCUNN error: %s is not implemented in this build\n", name);
}

// ---- element types of the hot path ---------------------------------------------------------------------
// The reference instantiates every entry point for float and double (THCGenerateFloatTypes.h); here the hot-path
// wrappers below are templates over one of these two descriptions: element type, `accreal` of the binding
// (THCUNN.lua:48,54), tensor struct, and the flat entry points that do the work.
struct RealFloat {
    typedef float real;
    typedef float accreal;
    typedef THCudaTensor tensor;
    static constexpr auto dwconv_forward = &cunn_b200_dwconv_forward;
    static constexpr auto dwconv_grad_input = &cunn_b200_dwconv_grad_input;
    static constexpr auto dwconv_acc_grad_workspace = &cunn_b200_dwconv_acc_grad_workspace;
    static constexpr auto dwconv_acc_grad = &cunn_b200_dwconv_acc_grad;
    static constexpr auto convmm_forward = &cunn_b200_convmm_forward;
    static constexpr auto convmm_grad_input = &cunn_b200_convmm_grad_input;
    static constexpr auto convmm_acc_grad_workspace = &cunn_b200_convmm_acc_grad_workspace;
    static constexpr auto convmm_acc_grad = &cunn_b200_convmm_acc_grad;
    static constexpr auto batchnorm_workspace = &cunn_b200_batchnorm_workspace;
    static constexpr auto batchnorm_forward = &cunn_b200_batchnorm_forward;
    static constexpr auto batchnorm_backward = &cunn_b200_batchnorm_backward;
    static constexpr auto maxpool_forward = &cunn_b200_maxpool_forward;
    static constexpr auto maxpool_backward = &cunn_b200_maxpool_backward;
};
struct RealDouble {
    typedef double real;
    typedef double accreal;
    typedef THCudaDoubleTensor tensor;
    static constexpr auto dwconv_forward = &cunn_b200_double_dwconv_forward;
    static constexpr auto dwconv_grad_input = &cunn_b200_double_dwconv_grad_input;
    static constexpr auto dwconv_acc_grad_workspace = &cunn_b200_double_dwconv_acc_grad_workspace;
    static constexpr auto dwconv_acc_grad = &cunn_b200_double_dwconv_acc_grad;
    static constexpr auto convmm_forward = &cunn_b200_double_convmm_forward;
    static constexpr auto convmm_grad_input = &cunn_b200_double_convmm_grad_input;
    static constexpr auto convmm_acc_grad_workspace = &cunn_b200_double_convmm_acc_grad_workspace;
    static constexpr auto convmm_acc_grad = &cunn_b200_double_convmm_acc_grad;
    static constexpr auto batchnorm_workspace = &cunn_b200_double_batchnorm_workspace;
    static constexpr auto batchnorm_forward = &cunn_b200_double_batchnorm_forward;
    static constexpr auto batchnorm_backward = &cunn_b200_double_batchnorm_backward;
    static constexpr auto maxpool_forward = &cunn_b200_double_maxpool_forward;
    static constexpr auto maxpool_backward = &cunn_b200_double_maxpool_backward;
};

// ---- SpatialDepthWiseConvolution -------------------------------------------------------------------
// Shape rules of lib/THCUNN/generic/SpatialDepthWiseConvolution.cu:5-56.  A 2-D weight [M, C*kH*kW] is
// given its 4-D shape in place, as the reference does (:76-80).
template <class Tensor>
static bool dw_prepare(THCState *s, Tensor *input, Tensor *gradOutput, Tensor *weight, Tensor *bias,
                       int kH, int kW, int dH, int dW, int padH, int padW, long *N, long *C, long *M, long *H, long *W,
                       long *oH, long *oW)
{
    if (!(kW > 0 && kH > 0)) { raise(s, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW); return false; }
    if (!(dW > 0 && dH > 0)) { raise(s, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW); return false; }
    if (weight->nDimension == 2) {
        const long m = weight->size[0], c = weight->size[1] / (kH * kW);
        const long sz[4] = {m, c, kH, kW};
        if (!tensor_resize(s, weight, 4, sz, 4)) return false;
    }
    if (weight->nDimension != 4) { raise(s, "2D or 4D weight tensor expected, but got: %s", size_desc(weight).c_str()); return false; }
    if (bias && !(check_dim_size(s, bias, "bias", 2, 0, weight->size[0]) && check_dim_size(s, bias, "bias", 2, 1, weight->size[1]))) return false;
    const int nd = input->nDimension;
    if (nd != 3 && nd != 4) { raise(s, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str()); return false; }
    const int b = nd == 4;
    *M = weight->size[0]; *C = weight->size[1];
    *N = b ? input->size[0] : 1; *H = input->size[b + 1]; *W = input->size[b + 2];
    *oH = (*H + 2 * padH - kH) / dH + 1; *oW = (*W + 2 * padW - kW) / dW + 1;
    if (*oW < 1 || *oH < 1) {
        raise(s, "Given input size: (%ld x %ld x %ld). Calculated output size: (%ld x %ld x %ld). Output size is too small", *C, *H, *W, *M * *C, *oH, *oW);
        return false;
    }
    if (!check_dim_size(s, input, "input", nd, b, *C)) return false;
    if (gradOutput) {
        // the reference views gradOutput as [N, C, M, oH, oW]; here the 4-D [N, C*M, oH, oW] form is checked
        if (gradOutput->nDimension != nd || gradOutput->size[b] != *C * *M || gradOutput->size[b + 1] != *oH || gradOutput->size[b + 2] != *oW) {
            raise(s, "Need gradOutput of shape [.. x %ld x %ld x %ld] but got gradOutput to be of shape: %s", *C * *M, *oH, *oW, size_desc(gradOutput).c_str());
            return false;
        }
    }
    return true;
}

template <class R>
static void hot_SpatialDepthWiseConvolution_updateOutput(
    THCState *s, typename R::tensor *input, typename R::tensor *output, typename R::tensor *weight, typename R::tensor *bias, typename R::tensor *,
    typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH)
{
    long N, C, M, H, W, oH, oW;
    if (!dw_prepare<typename R::tensor>(s, input, nullptr, weight, bias, kH, kW, dH, dW, padH, padW, &N, &C, &M, &H, &W, &oH, &oW)) return;
    typename R::tensor *x = new_contiguous(s, input, (int)sizeof(typename R::real)), *w = new_contiguous(s, weight, (int)sizeof(typename R::real)), *b = bias ? new_contiguous(s, bias, (int)sizeof(typename R::real)) : nullptr;
    if (x && w && (!bias || b)) {
        const long sz4[4] = {N, C * M, oH, oW};
        if (tensor_resize(s, output, 4, sz4, (int)sizeof(typename R::real))) {
            TH_CALL(s, R::dwconv_forward(tdata<typename R::real>(x), tdata<typename R::real>(w), tdata<typename R::real>(b), tdata<typename R::real>(output), (int)N,
                                                (int)C, (int)H, (int)W, (int)M, kH, kW, dH, dW, padH, padW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, output, 3, sz4 + 1, (int)sizeof(typename R::real));
        }
    }
done:
    tensor_free(s, x); tensor_free(s, w); tensor_free(s, b);
}

template <class R>
static void hot_SpatialDepthWiseConvolution_updateGradInput(
    THCState *s, typename R::tensor *input, typename R::tensor *gradOutput, typename R::tensor *gradInput, typename R::tensor *weight,
    typename R::tensor *, typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH)
{
    long N, C, M, H, W, oH, oW;
    if (!dw_prepare<typename R::tensor>(s, input, gradOutput, weight, nullptr, kH, kW, dH, dW, padH, padW, &N, &C, &M, &H, &W, &oH, &oW)) return;
    // unlike the reference (which views a strided gradOutput as if it were contiguous), gy is made contiguous
    typename R::tensor *gy = new_contiguous(s, gradOutput, (int)sizeof(typename R::real)), *w = new_contiguous(s, weight, (int)sizeof(typename R::real));
    if (gy && w) {
        const long sz4[4] = {N, C, H, W};
        if (tensor_resize(s, gradInput, 4, sz4, (int)sizeof(typename R::real))) {
            TH_CALL(s, R::dwconv_grad_input(tdata<typename R::real>(gy), tdata<typename R::real>(w), tdata<typename R::real>(gradInput), (int)N, (int)C,
                                                   (int)H, (int)W, (int)M, kH, kW, dH, dW, padH, padW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, gradInput, 3, sz4 + 1, (int)sizeof(typename R::real));
        }
    }
done:
    tensor_free(s, gy); tensor_free(s, w);
}

template <class R>
static void hot_SpatialDepthWiseConvolution_accGradParameters(
    THCState *s, typename R::tensor *input, typename R::tensor *gradOutput, typename R::tensor *gradWeight, typename R::tensor *gradBias,
    typename R::tensor *, typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH, typename R::accreal scale)
{
    long N, C, M, H, W, oH, oW;
    if (!dw_prepare<typename R::tensor>(s, input, gradOutput, gradWeight, gradBias, kH, kW, dH, dW, padH, padW, &N, &C, &M, &H, &W, &oH, &oW)) return;
    TH_CHECK(s, is_contiguous(gradWeight) && (!gradBias || is_contiguous(gradBias)), "gradWeight and gradBias have to be contiguous");
    typename R::tensor *x = new_contiguous(s, input, (int)sizeof(typename R::real)), *gy = new_contiguous(s, gradOutput, (int)sizeof(typename R::real));
    if (x && gy) {
        const size_t need = R::dwconv_acc_grad_workspace((int)N, (int)C, (int)H, (int)W, (int)M, kH, kW, dH, dW, padH, padW);
        void *ws = need ? state_scratch(s, 1, need) : nullptr;
        if (!need || ws)
            TH_CALL(s, R::dwconv_acc_grad(tdata<typename R::real>(x), tdata<typename R::real>(gy), tdata<typename R::real>(gradWeight), tdata<typename R::real>(gradBias),
                                                 (int)N, (int)C, (int)H, (int)W, (int)M, kH, kW, dH, dW, padH, padW, scale, ws,
                                                 state_scratch_bytes(s, 1), state_stream(s)));
    }
done:
    tensor_free(s, x); tensor_free(s, gy);
}

// ---- SpatialConvolutionMM ----------------------------------------------------------------------------
// Shape rules of lib/THCUNN/generic/SpatialConvolutionMM.cu:5-56; the weight must be contiguous (:74) and
// may be 2-D [K, C*kH*kW] or 4-D.
template <class Tensor>
static bool mm_prepare(THCState *s, Tensor *input, Tensor *gradOutput, Tensor *weight, Tensor *bias,
                       int kH, int kW, int dH, int dW, int padH, int padW, long *N, long *C, long *K, long *H, long *W,
                       long *oH, long *oW, int dilH = 1, int dilW = 1)
{
    if (!(dilW > 0 && dilH > 0)) { raise(s, "dilation should be greater than zero, but got dilationH: %d, dilationW: %d", dilH, dilW); return false; }
    if (!(kW > 0 && kH > 0)) { raise(s, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW); return false; }
    if (!(dW > 0 && dH > 0)) { raise(s, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW); return false; }
    if (!is_contiguous(weight)) { raise(s, "weight tensor has to be contiguous"); return false; }
    if (bias && !is_contiguous(bias)) { raise(s, "bias tensor has to be contiguous"); return false; }
    if (weight->nDimension != 2 && weight->nDimension != 4) { raise(s, "2D or 4D weight tensor expected, but got: %s", size_desc(weight).c_str()); return false; }
    *K = weight->size[0];
    *C = weight->nDimension == 2 ? weight->size[1] / (kH * kW) : weight->size[1];
    if (bias && !check_dim_size(s, bias, "bias", 1, 0, *K)) return false;
    const int nd = input->nDimension;
    if (nd != 3 && nd != 4) { raise(s, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str()); return false; }
    const int b = nd == 4;
    *N = b ? input->size[0] : 1; *H = input->size[b + 1]; *W = input->size[b + 2];
    *oH = (*H + 2 * padH - (dilH * (kH - 1) + 1)) / dH + 1; *oW = (*W + 2 * padW - (dilW * (kW - 1) + 1)) / dW + 1;
    if (*oW < 1 || *oH < 1) {
        raise(s, "Given input size: (%ld x %ld x %ld). Calculated output size: (%ld x %ld x %ld). Output size is too small", *C, *H, *W, *K, *oH, *oW);
        return false;
    }
    if (!check_dim_size(s, input, "input", nd, b, *C)) return false;
    if (gradOutput && !(check_dim_size(s, gradOutput, "gradOutput", nd, b, *K) && check_dim_size(s, gradOutput, "gradOutput", nd, b + 1, *oH) &&
                        check_dim_size(s, gradOutput, "gradOutput", nd, b + 2, *oW))) return false;
    return true;
}

template <class R>
static void hot_SpatialConvolutionMM_updateOutput(
    THCState *s, typename R::tensor *input, typename R::tensor *output, typename R::tensor *weight, typename R::tensor *bias, typename R::tensor *,
    typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<typename R::tensor>(s, input, nullptr, weight, bias, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW)) return;
    typename R::tensor *x = new_contiguous(s, input, (int)sizeof(typename R::real));
    if (x) {
        const long sz4[4] = {N, K, oH, oW};
        if (tensor_resize(s, output, 4, sz4, (int)sizeof(typename R::real))) {
            TH_CALL(s, R::convmm_forward(tdata<typename R::real>(x), tdata<typename R::real>(weight), bias ? tdata<typename R::real>(bias) : nullptr, tdata<typename R::real>(output),
                                                (int)N, (int)C, (int)H, (int)W, (int)K, kH, kW, dH, dW, padH, padW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, output, 3, sz4 + 1, (int)sizeof(typename R::real));
        }
    }
done:
    tensor_free(s, x);
}

template <class R>
static void hot_SpatialConvolutionMM_updateGradInput(
    THCState *s, typename R::tensor *input, typename R::tensor *gradOutput, typename R::tensor *gradInput, typename R::tensor *weight,
    typename R::tensor *, typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<typename R::tensor>(s, input, gradOutput, weight, nullptr, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW)) return;
    typename R::tensor *gy = new_contiguous(s, gradOutput, (int)sizeof(typename R::real));
    if (gy) {
        const long sz4[4] = {N, C, H, W};
        if (tensor_resize(s, gradInput, 4, sz4, (int)sizeof(typename R::real))) {
            TH_CALL(s, R::convmm_grad_input(tdata<typename R::real>(gy), tdata<typename R::real>(weight), tdata<typename R::real>(gradInput), (int)N, (int)C, (int)H,
                                                   (int)W, (int)K, kH, kW, dH, dW, padH, padW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, gradInput, 3, sz4 + 1, (int)sizeof(typename R::real));
        }
    }
done:
    tensor_free(s, gy);
}

template <class R>
static void hot_SpatialConvolutionMM_accGradParameters(
    THCState *s, typename R::tensor *input, typename R::tensor *gradOutput, typename R::tensor *gradWeight, typename R::tensor *gradBias,
    typename R::tensor *, typename R::tensor *, int kW, int kH, int dW, int dH, int padW, int padH, typename R::accreal scale)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<typename R::tensor>(s, input, gradOutput, gradWeight, gradBias, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW)) return;
    typename R::tensor *x = new_contiguous(s, input, (int)sizeof(typename R::real)), *gy = new_contiguous(s, gradOutput, (int)sizeof(typename R::real));
    if (x && gy) {
        const size_t need = R::convmm_acc_grad_workspace((int)N, (int)C, (int)H, (int)W, (int)K, kH, kW, dH, dW, padH, padW);
        void *ws = need ? state_scratch(s, 0, need) : nullptr;
        if (!need || ws)
            TH_CALL(s, R::convmm_acc_grad(tdata<typename R::real>(x), tdata<typename R::real>(gy), tdata<typename R::real>(gradWeight), gradBias ? tdata<typename R::real>(gradBias) : nullptr,
                                                 (int)N, (int)C, (int)H, (int)W, (int)K, kH, kW, dH, dW, padH, padW, scale, ws,
                                                 state_scratch_bytes(s, 0), state_stream(s)));
    }
done:
    tensor_free(s, x); tensor_free(s, gy);
}

// ---- SpatialDilatedConvolution (generic/SpatialDilatedConvolution.cu; decl generic/THCUNN.h:727-764): the same
// implicit GEMM with taps dilation apart.  `columns` / `ones` / `gradColumns` are accepted and left untouched.
extern "C" CUNN_API void THNN_CudaSpatialDilatedConvolution_updateOutput(
    THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *,
    THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<THCudaTensor>(s, input, nullptr, weight, bias, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW, dilationH, dilationW)) return;
    THCudaTensor *x = new_contiguous(s, input);
    if (x) {
        const long sz4[4] = {N, K, oH, oW};
        if (tensor_resize(s, output, 4, sz4, 4)) {
            TH_CALL(s, cunn_b200_dilated_conv_forward(tdata<float>(x), tdata<float>(weight), bias ? tdata<float>(bias) : nullptr,
                                                      tdata<float>(output), (int)N, (int)C, (int)H, (int)W, (int)K, kH, kW, dH, dW,
                                                      padH, padW, dilationH, dilationW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, output, 3, sz4 + 1, 4);
        }
    }
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaSpatialDilatedConvolution_updateGradInput(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<THCudaTensor>(s, input, gradOutput, weight, nullptr, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW, dilationH, dilationW)) return;
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy) {
        const long sz4[4] = {N, C, H, W};
        if (tensor_resize(s, gradInput, 4, sz4, 4)) {
            TH_CALL(s, cunn_b200_dilated_conv_grad_input(tdata<float>(gy), tdata<float>(weight), tdata<float>(gradInput), (int)N, (int)C,
                                                         (int)H, (int)W, (int)K, kH, kW, dH, dW, padH, padW, dilationH, dilationW,
                                                         state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, gradInput, 3, sz4 + 1, 4);
        }
    }
done:
    tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaSpatialDilatedConvolution_accGradParameters(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *, THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH,
    float scale)
{
    long N, C, K, H, W, oH, oW;
    if (!mm_prepare<THCudaTensor>(s, input, gradOutput, gradWeight, gradBias, kH, kW, dH, dW, padH, padW, &N, &C, &K, &H, &W, &oH, &oW, dilationH, dilationW)) return;
    THCudaTensor *x = new_contiguous(s, input), *gy = new_contiguous(s, gradOutput);
    if (x && gy) {
        const size_t need = cunn_b200_dilated_conv_acc_grad_workspace((int)N, (int)C, (int)H, (int)W, (int)K, kH, kW, dH, dW, padH, padW,
                                                                       dilationH, dilationW);
        void *ws = need ? state_scratch(s, 0, need) : nullptr;
        if (!need || ws)
            TH_CALL(s, cunn_b200_dilated_conv_acc_grad(tdata<float>(x), tdata<float>(gy), tdata<float>(gradWeight),
                                                       gradBias ? tdata<float>(gradBias) : nullptr, (int)N, (int)C, (int)H, (int)W, (int)K,
                                                       kH, kW, dH, dW, padH, padW, dilationH, dilationW, scale, ws, need, state_stream(s)));
    }
done:
    tensor_free(s, x);
    tensor_free(s, gy);
}

// ---- SpatialFullDilatedConvolution / SpatialFullConvolution (transposed convolution) ----------------------
// Shape rules of lib/THCUNN/generic/SpatialFullDilatedConvolution.cu:5-66: weight [nInputPlane, nOutputPlane, kH, kW]
// (or 2-D [nInputPlane, nOutputPlane*kH*kW]), bias [nOutputPlane].
static bool full_prepare(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *weight, THCudaTensor *bias,
                         int kH, int kW, int dH, int dW, int padH, int padW, int dilH, int dilW, int adjH, int adjW, long *N,
                         long *P, long *Q, long *H, long *W, long *OH, long *OW)
{
    if (!(kW > 0 && kH > 0)) { raise(s, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW); return false; }
    if (!(dW > 0 && dH > 0)) { raise(s, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW); return false; }
    if (!(dilW > 0 && dilH > 0)) { raise(s, "dilation should be greater than zero, but got dilationH: %d, dilationW: %d", dilH, dilW); return false; }
    if (!((adjW < dW || adjW < dilW) && (adjH < dH || adjH < dilH))) {
        raise(s, "output padding must be smaller than either stride or dilation, but got adjH: %d adjW: %d dH: %d dW: %d dilationH: %d dilationW: %d",
              adjH, adjW, dH, dW, dilH, dilW);
        return false;
    }
    if (!is_contiguous(weight)) { raise(s, "weight tensor has to be contiguous"); return false; }
    if (bias && !is_contiguous(bias)) { raise(s, "bias tensor has to be contiguous"); return false; }
    if (weight->nDimension != 2 && weight->nDimension != 4) { raise(s, "2D or 4D weight tensor expected, but got: %s", size_desc(weight).c_str()); return false; }
    *P = weight->size[0];
    *Q = weight->nDimension == 2 ? weight->size[1] / (kH * kW) : weight->size[1];
    if (bias && !check_dim_size(s, bias, "bias", 1, 0, *Q)) return false;
    const int nd = input->nDimension;
    if (nd != 3 && nd != 4) { raise(s, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str()); return false; }
    const int b = nd == 4;
    *N = b ? input->size[0] : 1; *H = input->size[b + 1]; *W = input->size[b + 2];
    *OH = (*H - 1) * dH - 2 * padH + (dilH * (kH - 1) + 1) + adjH;
    *OW = (*W - 1) * dW - 2 * padW + (dilW * (kW - 1) + 1) + adjW;
    if (*OW < 1 || *OH < 1) {
        raise(s, "Given input size: (%ld x %ld x %ld). Calculated output size: (%ld x %ld x %ld). Output size is too small", *P, *H, *W, *Q, *OH, *OW);
        return false;
    }
    if (!check_dim_size(s, input, "input", nd, b, *P)) return false;
    if (gradOutput && !(check_dim_size(s, gradOutput, "gradOutput", nd, b, *Q) && check_dim_size(s, gradOutput, "gradOutput", nd, b + 1, *OH) &&
                        check_dim_size(s, gradOutput, "gradOutput", nd, b + 2, *OW))) return false;
    return true;
}

extern "C" CUNN_API void THNN_CudaSpatialFullDilatedConvolution_updateOutput(
    THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *,
    THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH, int adjW, int adjH)
{
    long N, P, Q, H, W, OH, OW;
    if (!full_prepare(s, input, nullptr, weight, bias, kH, kW, dH, dW, padH, padW, dilationH, dilationW, adjH, adjW, &N, &P, &Q, &H, &W, &OH, &OW)) return;
    THCudaTensor *x = new_contiguous(s, input);
    if (x) {
        const long sz4[4] = {N, Q, OH, OW};
        if (tensor_resize(s, output, 4, sz4, 4)) {
            TH_CALL(s, cunn_b200_full_conv_forward(tdata<float>(x), tdata<float>(weight), bias ? tdata<float>(bias) : nullptr,
                                                   tdata<float>(output), (int)N, (int)P, (int)H, (int)W, (int)Q, kH, kW, dH, dW, padH,
                                                   padW, dilationH, dilationW, adjH, adjW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, output, 3, sz4 + 1, 4);
        }
    }
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaSpatialFullDilatedConvolution_updateGradInput(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH, int adjW, int adjH)
{
    long N, P, Q, H, W, OH, OW;
    if (!full_prepare(s, input, gradOutput, weight, nullptr, kH, kW, dH, dW, padH, padW, dilationH, dilationW, adjH, adjW, &N, &P, &Q, &H, &W, &OH, &OW)) return;
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy) {
        const long sz4[4] = {N, P, H, W};
        if (tensor_resize(s, gradInput, 4, sz4, 4)) {
            TH_CALL(s, cunn_b200_full_conv_grad_input(tdata<float>(gy), tdata<float>(weight), tdata<float>(gradInput), (int)N, (int)P,
                                                      (int)H, (int)W, (int)Q, kH, kW, dH, dW, padH, padW, dilationH, dilationW, adjH,
                                                      adjW, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, gradInput, 3, sz4 + 1, 4);
        }
    }
done:
    tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaSpatialFullDilatedConvolution_accGradParameters(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *, THCudaTensor *, int kW, int kH, int dW, int dH, int padW, int padH, int dilationW, int dilationH,
    int adjW, int adjH, float scale)
{
    long N, P, Q, H, W, OH, OW;
    if (!full_prepare(s, input, gradOutput, gradWeight, gradBias, kH, kW, dH, dW, padH, padW, dilationH, dilationW, adjH, adjW, &N, &P, &Q, &H, &W, &OH, &OW)) return;
    THCudaTensor *x = new_contiguous(s, input), *gy = new_contiguous(s, gradOutput);
    if (x && gy) {
        const size_t need = cunn_b200_full_conv_acc_grad_workspace((int)N, (int)P, (int)H, (int)W, (int)Q, kH, kW, dH, dW, padH, padW,
                                                                    dilationH, dilationW, adjH, adjW);
        void *ws = need ? state_scratch(s, 0, need) : nullptr;
        if (!need || ws)
            TH_CALL(s, cunn_b200_full_conv_acc_grad(tdata<float>(x), tdata<float>(gy), tdata<float>(gradWeight),
                                                    gradBias ? tdata<float>(gradBias) : nullptr, (int)N, (int)P, (int)H, (int)W, (int)Q,
                                                    kH, kW, dH, dW, padH, padW, dilationH, dilationW, adjH, adjW, scale, ws, need,
                                                    state_stream(s)));
    }
done:
    tensor_free(s, x);
    tensor_free(s, gy);
}

// SpatialFullConvolution is the same operator with dilation 1 (lib/THCUNN/generic/SpatialFullConvolution.cu).
extern "C" CUNN_API void THNN_CudaSpatialFullConvolution_updateOutput(
    THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *columns,
    THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH)
{
    THNN_CudaSpatialFullDilatedConvolution_updateOutput(s, input, output, weight, bias, columns, ones, kW, kH, dW, dH, padW, padH, 1, 1,
                                                        adjW, adjH);
}

extern "C" CUNN_API void THNN_CudaSpatialFullConvolution_updateGradInput(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight,
    THCudaTensor *gradColumns, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH)
{
    THNN_CudaSpatialFullDilatedConvolution_updateGradInput(s, input, gradOutput, gradInput, weight, gradColumns, kW, kH, dW, dH, padW,
                                                           padH, 1, 1, adjW, adjH);
}

extern "C" CUNN_API void THNN_CudaSpatialFullConvolution_accGradParameters(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias,
    THCudaTensor *columns, THCudaTensor *ones, int kW, int kH, int dW, int dH, int padW, int padH, int adjW, int adjH, float scale)
{
    THNN_CudaSpatialFullDilatedConvolution_accGradParameters(s, input, gradOutput, gradWeight, gradBias, columns, ones, kW, kH, dW, dH,
                                                             padW, padH, 1, 1, adjW, adjH, scale);
}

// ---- BatchNormalization --------------------------------------------------------------------------------
// Any [N, C, ...] input is viewed as [N, C, S] (lib/THCUNN/generic/BatchNormalization.cu:8-32).
template <class Tensor>
static bool bn_dims(THCState *s, const Tensor *t, long *N, long *C, long *S)
{
    if (t->nDimension < 2) { raise(s, "batch normalisation expects at least 2 dimensions, got: %s", size_desc(t).c_str()); return false; }
    *N = t->size[0]; *C = t->size[1]; *S = 1;
    for (int i = 2; i < t->nDimension; ++i) *S *= t->size[i];
    return true;
}

template <class R>
static void hot_BatchNormalization_updateOutput(
    THCState *s, typename R::tensor *input_, typename R::tensor *output_, typename R::tensor *weight_, typename R::tensor *bias_,
    typename R::tensor *runningMean_, typename R::tensor *runningVar_, typename R::tensor *saveMean_, typename R::tensor *saveStd_, bool train,
    double momentum, double eps)
{
    long N, C, S;
    if (!bn_dims<typename R::tensor>(s, input_, &N, &C, &S)) return;
    typename R::tensor *x = new_contiguous(s, input_, (int)sizeof(typename R::real));
    if (x && tensor_resize(s, output_, input_->nDimension, input_->size, (int)sizeof(typename R::real))) {
        const long c1[1] = {C};
        if (!train || (tensor_resize(s, saveMean_, 1, c1, (int)sizeof(typename R::real)) && tensor_resize(s, saveStd_, 1, c1, (int)sizeof(typename R::real)))) {
            void *ws = state_scratch(s, 2, R::batchnorm_workspace((int)N, (int)C));
            if (ws)
                TH_CALL(s, R::batchnorm_forward(tdata<typename R::real>(x), tdata<typename R::real>(output_), weight_ ? tdata<typename R::real>(weight_) : nullptr,
                                                       bias_ ? tdata<typename R::real>(bias_) : nullptr, tdata<typename R::real>(runningMean_), tdata<typename R::real>(runningVar_),
                                                       tdata<typename R::real>(saveMean_), tdata<typename R::real>(saveStd_), (int)N, (int)C, (int)S, train ? 1 : 0,
                                                       momentum, eps, ws, state_scratch_bytes(s, 2), state_stream(s)));
        }
    }
done:
    tensor_free(s, x);
}

template <class R>
static void hot_BatchNormalization_backward(
    THCState *s, typename R::tensor *input_, typename R::tensor *gradOutput_, typename R::tensor *gradInput_, typename R::tensor *gradWeight_,
    typename R::tensor *gradBias_, typename R::tensor *weight_, typename R::tensor *runningMean_, typename R::tensor *runningVar_,
    typename R::tensor *saveMean_, typename R::tensor *saveStd_, bool train, double scale, double eps)
{
    long N, C, S;
    if (!bn_dims<typename R::tensor>(s, input_, &N, &C, &S)) return;
    TH_CHECK(s, nelem(gradOutput_) == nelem(input_), "input and gradOutput have different number of elements: input%s, gradOutput%s",
             size_desc(input_).c_str(), size_desc(gradOutput_).c_str());
    typename R::tensor *x = new_contiguous(s, input_, (int)sizeof(typename R::real)), *gy = new_contiguous(s, gradOutput_, (int)sizeof(typename R::real));
    if (x && gy && (!gradInput_ || tensor_resize(s, gradInput_, input_->nDimension, input_->size, (int)sizeof(typename R::real)))) {
        void *ws = state_scratch(s, 2, R::batchnorm_workspace((int)N, (int)C));
        if (ws)
            TH_CALL(s, R::batchnorm_backward(tdata<typename R::real>(x), tdata<typename R::real>(gy), gradInput_ ? tdata<typename R::real>(gradInput_) : nullptr,
                                                    gradWeight_ ? tdata<typename R::real>(gradWeight_) : nullptr, gradBias_ ? tdata<typename R::real>(gradBias_) : nullptr,
                                                    weight_ ? tdata<typename R::real>(weight_) : nullptr, tdata<typename R::real>(runningMean_), tdata<typename R::real>(runningVar_),
                                                    tdata<typename R::real>(saveMean_), tdata<typename R::real>(saveStd_), (int)N, (int)C, (int)S, train ? 1 : 0, scale, eps,
                                                    ws, state_scratch_bytes(s, 2), state_stream(s)));
    }
done:
    tensor_free(s, x); tensor_free(s, gy);
}

// ---- SpatialMaxPooling ------------------------------------------------------------------------------------
template <class R>
static void hot_SpatialMaxPooling_updateOutput(THCState *s, typename R::tensor *input, typename R::tensor *output,
                                                                 THCudaLongTensor *indices, int kW, int kH, int dW, int dH,
                                                                 int padW, int padH, bool ceil_mode)
{
    const int nd = input->nDimension;
    TH_CHECK(s, nd == 3 || nd == 4, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str());
    TH_CHECK(s, kW > 0 && kH > 0, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW);
    TH_CHECK(s, dW > 0 && dH > 0, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW);
    const int b = nd == 4;
    const long N = b ? input->size[0] : 1, C = input->size[b], H = input->size[b + 1], W = input->size[b + 2];
    const long oH = cunn_b200_maxpool_out_size((int)H, kH, dH, padH, 1, ceil_mode), oW = cunn_b200_maxpool_out_size((int)W, kW, dW, padW, 1, ceil_mode);
    typename R::tensor *x = new_contiguous(s, input, (int)sizeof(typename R::real));
    if (x) {
        const long sz4[4] = {N, C, oH > 0 ? oH : 0, oW > 0 ? oW : 0};
        if (oH < 1 || oW < 1 || (tensor_resize(s, output, 4, sz4, (int)sizeof(typename R::real)) && tensor_resize(s, indices, 4, sz4, 8))) {
            TH_CALL(s, R::maxpool_forward(tdata<typename R::real>(x), tdata<typename R::real>(output), tdata<int64_t>(indices), (int)N, (int)C, (int)H, (int)W, kH,
                                                 kW, dH, dW, padH, padW, 1, 1, ceil_mode, state_stream(s)));
            if (nd == 3) tensor_resize(s, output, 3, sz4 + 1, (int)sizeof(typename R::real));   // indices stay 4-D, as in the reference
        }
    }
done:
    tensor_free(s, x);
}

template <class R>
static void hot_SpatialMaxPooling_updateGradInput(THCState *s, typename R::tensor *input, typename R::tensor *gradOutput,
                                                                    typename R::tensor *gradInput, THCudaLongTensor *indices, int kW,
                                                                    int kH, int dW, int dH, int padW, int padH, bool ceil_mode)
{
    const int nd = input->nDimension;
    TH_CHECK(s, nd == 3 || nd == 4, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str());
    const int b = nd == 4;
    const long N = b ? input->size[0] : 1, C = input->size[b], H = input->size[b + 1], W = input->size[b + 2];
    const long oH = cunn_b200_maxpool_out_size((int)H, kH, dH, padH, 1, ceil_mode), oW = cunn_b200_maxpool_out_size((int)W, kW, dW, padW, 1, ceil_mode);
    TH_CHECK(s, gradOutput->nDimension == nd && gradOutput->size[b] == C && gradOutput->size[b + 1] == oH && gradOutput->size[b + 2] == oW,
             "Need gradOutput of dimension %d and shape [.. x %ld x %ld x %ld] but got gradOutput to be of shape: %s", nd, C, oH, oW,
             size_desc(gradOutput).c_str());
    TH_CHECK(s, nelem(indices) == nelem(gradOutput) && is_contiguous(indices), "indices and gradOutput shapes do not match");
    typename R::tensor *gy = new_contiguous(s, gradOutput, (int)sizeof(typename R::real));
    if (gy && tensor_resize(s, gradInput, nd, input->size, (int)sizeof(typename R::real)))
        TH_CALL(s, R::maxpool_backward(tdata<typename R::real>(gy), tdata<int64_t>(indices), tdata<typename R::real>(gradInput), (int)N, (int)C, (int)H, (int)W,
                                              kH, kW, dH, dW, padH, padW, 1, 1, ceil_mode, state_stream(s)));
done:
    tensor_free(s, gy);
}

// ---- exported entry points of the hot path, float and double ----------------------------------------------------
extern "C" CUNN_API void THNN_CudaSpatialDepthWiseConvolution_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialDepthWiseConvolution_updateOutput<RealFloat>(s, input, output, weight, bias, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_updateOutput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaDoubleTensor *weight, THCudaDoubleTensor *bias, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialDepthWiseConvolution_updateOutput<RealDouble>(s, input, output, weight, bias, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaSpatialDepthWiseConvolution_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialDepthWiseConvolution_updateGradInput<RealFloat>(s, input, gradOutput, gradInput, weight, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_updateGradInput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaDoubleTensor *weight, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialDepthWiseConvolution_updateGradInput<RealDouble>(s, input, gradOutput, gradInput, weight, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaSpatialDepthWiseConvolution_accGradParameters(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH, float scale)
{
    hot_SpatialDepthWiseConvolution_accGradParameters<RealFloat>(s, input, gradOutput, gradWeight, gradBias, unused5, unused6, kW, kH, dW, dH, padW, padH, scale);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialDepthWiseConvolution_accGradParameters(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradWeight, THCudaDoubleTensor *gradBias, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH, double scale)
{
    hot_SpatialDepthWiseConvolution_accGradParameters<RealDouble>(s, input, gradOutput, gradWeight, gradBias, unused5, unused6, kW, kH, dW, dH, padW, padH, scale);
}
extern "C" CUNN_API void THNN_CudaSpatialConvolutionMM_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialConvolutionMM_updateOutput<RealFloat>(s, input, output, weight, bias, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_updateOutput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaDoubleTensor *weight, THCudaDoubleTensor *bias, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialConvolutionMM_updateOutput<RealDouble>(s, input, output, weight, bias, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaSpatialConvolutionMM_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialConvolutionMM_updateGradInput<RealFloat>(s, input, gradOutput, gradInput, weight, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_updateGradInput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaDoubleTensor *weight, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH)
{
    hot_SpatialConvolutionMM_updateGradInput<RealDouble>(s, input, gradOutput, gradInput, weight, unused5, unused6, kW, kH, dW, dH, padW, padH);
}
extern "C" CUNN_API void THNN_CudaSpatialConvolutionMM_accGradParameters(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias, THCudaTensor *unused5, THCudaTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH, float scale)
{
    hot_SpatialConvolutionMM_accGradParameters<RealFloat>(s, input, gradOutput, gradWeight, gradBias, unused5, unused6, kW, kH, dW, dH, padW, padH, scale);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialConvolutionMM_accGradParameters(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradWeight, THCudaDoubleTensor *gradBias, THCudaDoubleTensor *unused5, THCudaDoubleTensor *unused6, int kW, int kH, int dW, int dH, int padW, int padH, double scale)
{
    hot_SpatialConvolutionMM_accGradParameters<RealDouble>(s, input, gradOutput, gradWeight, gradBias, unused5, unused6, kW, kH, dW, dH, padW, padH, scale);
}
extern "C" CUNN_API void THNN_CudaBatchNormalization_updateOutput(THCState *s, THCudaTensor *input_, THCudaTensor *output_, THCudaTensor *weight_, THCudaTensor *bias_, THCudaTensor *runningMean_, THCudaTensor *runningVar_, THCudaTensor *saveMean_, THCudaTensor *saveStd_, bool train, double momentum, double eps)
{
    hot_BatchNormalization_updateOutput<RealFloat>(s, input_, output_, weight_, bias_, runningMean_, runningVar_, saveMean_, saveStd_, train, momentum, eps);
}
extern "C" CUNN_API void THNN_CudaDoubleBatchNormalization_updateOutput(THCState *s, THCudaDoubleTensor *input_, THCudaDoubleTensor *output_, THCudaDoubleTensor *weight_, THCudaDoubleTensor *bias_, THCudaDoubleTensor *runningMean_, THCudaDoubleTensor *runningVar_, THCudaDoubleTensor *saveMean_, THCudaDoubleTensor *saveStd_, bool train, double momentum, double eps)
{
    hot_BatchNormalization_updateOutput<RealDouble>(s, input_, output_, weight_, bias_, runningMean_, runningVar_, saveMean_, saveStd_, train, momentum, eps);
}
extern "C" CUNN_API void THNN_CudaBatchNormalization_backward(THCState *s, THCudaTensor *input_, THCudaTensor *gradOutput_, THCudaTensor *gradInput_, THCudaTensor *gradWeight_, THCudaTensor *gradBias_, THCudaTensor *weight_, THCudaTensor *runningMean_, THCudaTensor *runningVar_, THCudaTensor *saveMean_, THCudaTensor *saveStd_, bool train, double scale, double eps)
{
    hot_BatchNormalization_backward<RealFloat>(s, input_, gradOutput_, gradInput_, gradWeight_, gradBias_, weight_, runningMean_, runningVar_, saveMean_, saveStd_, train, scale, eps);
}
extern "C" CUNN_API void THNN_CudaDoubleBatchNormalization_backward(THCState *s, THCudaDoubleTensor *input_, THCudaDoubleTensor *gradOutput_, THCudaDoubleTensor *gradInput_, THCudaDoubleTensor *gradWeight_, THCudaDoubleTensor *gradBias_, THCudaDoubleTensor *weight_, THCudaDoubleTensor *runningMean_, THCudaDoubleTensor *runningVar_, THCudaDoubleTensor *saveMean_, THCudaDoubleTensor *saveStd_, bool train, double scale, double eps)
{
    hot_BatchNormalization_backward<RealDouble>(s, input_, gradOutput_, gradInput_, gradWeight_, gradBias_, weight_, runningMean_, runningVar_, saveMean_, saveStd_, train, scale, eps);
}
extern "C" CUNN_API void THNN_CudaSpatialMaxPooling_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaLongTensor *indices, int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode)
{
    hot_SpatialMaxPooling_updateOutput<RealFloat>(s, input, output, indices, kW, kH, dW, dH, padW, padH, ceil_mode);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialMaxPooling_updateOutput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *output, THCudaLongTensor *indices, int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode)
{
    hot_SpatialMaxPooling_updateOutput<RealDouble>(s, input, output, indices, kW, kH, dW, dH, padW, padH, ceil_mode);
}
extern "C" CUNN_API void THNN_CudaSpatialMaxPooling_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaLongTensor *indices, int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode)
{
    hot_SpatialMaxPooling_updateGradInput<RealFloat>(s, input, gradOutput, gradInput, indices, kW, kH, dW, dH, padW, padH, ceil_mode);
}
extern "C" CUNN_API void THNN_CudaDoubleSpatialMaxPooling_updateGradInput(THCState *s, THCudaDoubleTensor *input, THCudaDoubleTensor *gradOutput, THCudaDoubleTensor *gradInput, THCudaLongTensor *indices, int kW, int kH, int dW, int dH, int padW, int padH, bool ceil_mode)
{
    hot_SpatialMaxPooling_updateGradInput<RealDouble>(s, input, gradOutput, gradInput, indices, kW, kH, dW, dH, padW, padH, ceil_mode);
}

// ---- SpatialConvolutionLocal (generic/SpatialConvolutionLocal.cu; decl generic/THCUNN.h:587-628) --------------------
// weight 3-D [oH*oW, K, C*kH*kW] or 6-D [oH, oW, K, C, kH, kW] (:58-77); bias [K, oH, oW]; finput / fgradInput are the
// reference's unfolded copies and are not used.
static bool local_prepare(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *weight, THCudaTensor *bias, int kH, int kW,
                          int dH, int dW, long inputHeight, long inputWidth, long outputHeight, long outputWidth, long *N, long *C, long *K)
{
    if (!(kW > 0 && kH > 0)) { raise(s, "kernel size should be greater than zero, but got kH: %d kW: %d", kH, kW); return false; }
    if (!(dW > 0 && dH > 0)) { raise(s, "stride should be greater than zero, but got dH: %d dW: %d", dH, dW); return false; }
    const int nd = input->nDimension;
    if (nd != 3 && nd != 4) { raise(s, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str()); return false; }
    if (weight->nDimension != 3 && weight->nDimension != 6) { raise(s, "weight tensor should be 3D or 6D - got %dD", weight->nDimension); return false; }
    if (!is_contiguous(weight)) { raise(s, "weight tensor has to be contiguous"); return false; }
    const bool six = weight->nDimension == 6;
    *K = six ? weight->size[2] : weight->size[1];
    const long R = six ? weight->size[3] * weight->size[4] * weight->size[5] : weight->size[2];
    const long Pw = six ? weight->size[0] * weight->size[1] : weight->size[0];
    *C = R / (kH * kW);
    if (Pw != outputHeight * outputWidth) { raise(s, "weight holds %ld output positions, expected %ld x %ld", Pw, outputHeight, outputWidth); return false; }
    if (bias && !(check_dim_size(s, bias, "bias", 3, 0, *K) && check_dim_size(s, bias, "bias", 3, 1, outputHeight) &&
                  check_dim_size(s, bias, "bias", 3, 2, outputWidth))) return false;
    const int b = nd == 4;
    *N = b ? input->size[0] : 1;
    if (!check_dim_size(s, input, "input", nd, b, *C)) return false;
    if (input->size[b + 1] != inputHeight || input->size[b + 2] != inputWidth) {
        raise(s, "input is %ld x %ld, the module was built for %ld x %ld", input->size[b + 1], input->size[b + 2], inputHeight, inputWidth);
        return false;
    }
    if (gradOutput && !(check_dim_size(s, gradOutput, "gradOutput", nd, b, *K) && check_dim_size(s, gradOutput, "gradOutput", nd, b + 1, outputHeight) &&
                        check_dim_size(s, gradOutput, "gradOutput", nd, b + 2, outputWidth))) return false;
    return true;
}

extern "C" CUNN_API void THNN_CudaSpatialConvolutionLocal_updateOutput(
    THCState *s, THCudaTensor *input, THCudaTensor *output, THCudaTensor *weight, THCudaTensor *bias, THCudaTensor *, THCudaTensor *, int kW,
    int kH, int dW, int dH, int padW, int padH, long inputWidth, long inputHeight, long outputWidth, long outputHeight)
{
    long N, C, K;
    if (!local_prepare(s, input, nullptr, weight, bias, kH, kW, dH, dW, inputHeight, inputWidth, outputHeight, outputWidth, &N, &C, &K)) return;
    THCudaTensor *x = new_contiguous(s, input), *b = bias ? new_contiguous(s, bias) : nullptr;
    if (x && (!bias || b)) {
        const long sz4[4] = {N, K, outputHeight, outputWidth};
        if (tensor_resize(s, output, 4, sz4, 4)) {
            TH_CALL(s, cunn_b200_local_conv_forward(tdata<float>(x), tdata<float>(weight), tdata<float>(b), tdata<float>(output), (int)N, (int)C,
                                                    (int)inputHeight, (int)inputWidth, (int)K, kH, kW, dH, dW, padH, padW, (int)outputHeight,
                                                    (int)outputWidth, state_stream(s)));
            if (input->nDimension == 3) tensor_resize(s, output, 3, sz4 + 1, 4);
        }
    }
done:
    tensor_free(s, x); tensor_free(s, b);
}

extern "C" CUNN_API void THNN_CudaSpatialConvolutionLocal_updateGradInput(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradInput, THCudaTensor *weight, THCudaTensor *, THCudaTensor *,
    int kW, int kH, int dW, int dH, int padW, int padH, long inputWidth, long inputHeight, long outputWidth, long outputHeight)
{
    long N, C, K;
    if (!local_prepare(s, input, gradOutput, weight, nullptr, kH, kW, dH, dW, inputHeight, inputWidth, outputHeight, outputWidth, &N, &C, &K)) return;
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy && tensor_resize(s, gradInput, input->nDimension, input->size, 4))
        TH_CALL(s, cunn_b200_local_conv_grad_input(tdata<float>(gy), tdata<float>(weight), tdata<float>(gradInput), (int)N, (int)C, (int)inputHeight,
                                                   (int)inputWidth, (int)K, kH, kW, dH, dW, padH, padW, (int)outputHeight, (int)outputWidth,
                                                   state_stream(s)));
done:
    tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaSpatialConvolutionLocal_accGradParameters(
    THCState *s, THCudaTensor *input, THCudaTensor *gradOutput, THCudaTensor *gradWeight, THCudaTensor *gradBias, THCudaTensor *, THCudaTensor *,
    int kW, int kH, int dW, int dH, int padW, int padH, long inputWidth, long inputHeight, long outputWidth, long outputHeight, float scale)
{
    long N, C, K;
    if (!local_prepare(s, input, gradOutput, gradWeight, gradBias, kH, kW, dH, dW, inputHeight, inputWidth, outputHeight, outputWidth, &N, &C, &K)) return;
    TH_CHECK(s, !gradBias || is_contiguous(gradBias), "gradBias has to be contiguous");
    THCudaTensor *x = new_contiguous(s, input), *gy = new_contiguous(s, gradOutput);
    if (x && gy)
        TH_CALL(s, cunn_b200_local_conv_acc_grad(tdata<float>(x), tdata<float>(gy), tdata<float>(gradWeight), gradBias ? tdata<float>(gradBias) : nullptr,
                                                 (int)N, (int)C, (int)inputHeight, (int)inputWidth, (int)K, kH, kW, dH, dW, padH, padW,
                                                 (int)outputHeight, (int)outputWidth, scale, state_stream(s)));
done:
    tensor_free(s, x); tensor_free(s, gy);
}

// ---- SpatialAdaptiveMaxPooling / SpatialAdaptiveAveragePooling (decl generic/THCUNN.h:520-546) ---------------------
static bool adaptive_dims(THCState *s, const THCudaTensor *input, long *planes, long *H, long *W)
{
    const int nd = input->nDimension;
    if (nd != 3 && nd != 4) { raise(s, "3D or 4D (batch mode) tensor expected for input, but got: %s", size_desc(input).c_str()); return false; }
    const int b = nd == 4;
    *planes = (b ? input->size[0] : 1) * input->size[b];
    *H = input->size[b + 1];
    *W = input->size[b + 2];
    return true;
}

extern "C" CUNN_API void THNN_CudaSpatialAdaptiveMaxPooling_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output,
                                                                         THCudaLongTensor *indices, int nOutputCols, int nOutputRows)
{
    long planes, H, W;
    if (!adaptive_dims(s, input, &planes, &H, &W)) return;
    const int b = input->nDimension == 4;
    THCudaTensor *x = new_contiguous(s, input);
    if (x) {
        const long osz[4] = {b ? input->size[0] : 0, input->size[b], nOutputRows, nOutputCols};
        const long isz[5] = {2, b ? input->size[0] : 0, input->size[b], nOutputRows, nOutputCols};
        const long isz3[4] = {2, input->size[b], nOutputRows, nOutputCols};
        // indices: [2, (N,) C, oH, oW] as the reference resizes them (generic/SpatialAdaptiveMaxPooling.cu:35,64)
        const bool ok = b ? (tensor_resize(s, output, 4, osz, 4) && tensor_resize(s, indices, 5, isz, 8))
                          : (tensor_resize(s, output, 3, osz + 1, 4) && tensor_resize(s, indices, 4, isz3, 8));
        if (ok)
            TH_CALL(s, cunn_b200_adaptive_maxpool_forward(tdata<float>(x), tdata<float>(output), tdata<int64_t>(indices), (int)planes, (int)H, (int)W,
                                                          nOutputRows, nOutputCols, state_stream(s)));
    }
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaSpatialAdaptiveMaxPooling_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput,
                                                                            THCudaTensor *gradInput, THCudaLongTensor *indices)
{
    long planes, H, W;
    if (!adaptive_dims(s, input, &planes, &H, &W)) return;
    const int b = input->nDimension == 4;
    TH_CHECK(s, gradOutput->nDimension == input->nDimension, "gradOutput must have input's number of dimensions");
    const long oH = gradOutput->size[b + 1], oW = gradOutput->size[b + 2];
    TH_CHECK(s, nelem(indices) == 2 * nelem(gradOutput) && is_contiguous(indices), "indices and gradOutput shapes do not match");
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy && tensor_resize(s, gradInput, input->nDimension, input->size, 4))
        TH_CALL(s, cunn_b200_adaptive_maxpool_backward(tdata<float>(gy), tdata<int64_t>(indices), tdata<float>(gradInput), (int)planes, (int)H, (int)W,
                                                       (int)oH, (int)oW, state_stream(s)));
done:
    tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaSpatialAdaptiveAveragePooling_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output,
                                                                             int nOutputCols, int nOutputRows)
{
    long planes, H, W;
    if (!adaptive_dims(s, input, &planes, &H, &W)) return;
    const int b = input->nDimension == 4;
    THCudaTensor *x = new_contiguous(s, input);
    if (x) {
        const long osz[4] = {b ? input->size[0] : 0, input->size[b], nOutputRows, nOutputCols};
        if (tensor_resize(s, output, b ? 4 : 3, b ? osz : osz + 1, 4))
            TH_CALL(s, cunn_b200_adaptive_avgpool_forward(tdata<float>(x), tdata<float>(output), (int)planes, (int)H, (int)W, nOutputRows,
                                                          nOutputCols, state_stream(s)));
    }
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaSpatialAdaptiveAveragePooling_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput,
                                                                                THCudaTensor *gradInput)
{
    long planes, H, W;
    if (!adaptive_dims(s, input, &planes, &H, &W)) return;
    const int b = input->nDimension == 4;
    TH_CHECK(s, gradOutput->nDimension == input->nDimension, "gradOutput must have input's number of dimensions");
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy && tensor_resize(s, gradInput, input->nDimension, input->size, 4))
        TH_CALL(s, cunn_b200_adaptive_avgpool_backward(tdata<float>(gy), tdata<float>(gradInput), (int)planes, (int)H, (int)W,
                                                       (int)gradOutput->size[b + 1], (int)gradOutput->size[b + 2], state_stream(s)));
done:
    tensor_free(s, gy);
}

// ---- support operators ---------------------------------------------------------------------------------------
extern "C" CUNN_API void THNN_CudaThreshold_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output, float threshold,
                                                         float val, bool inplace)
{
    if (inplace) {
        TH_CHECK(s, is_contiguous(input), "in-place Threshold needs a contiguous input");
        if (cunn_b200_threshold_forward(tdata<float>(input), tdata<float>(input), nelem(input), threshold, val, state_stream(s))) raise(s, "%s", cunn_b200_last_error());
        // the reference makes output share input's storage (THCTensor_set); callers keep using `input`
        return;
    }
    THCudaTensor *x = new_contiguous(s, input);
    if (x && tensor_resize(s, output, input->nDimension, input->size, 4))
        TH_CALL(s, cunn_b200_threshold_forward(tdata<float>(x), tdata<float>(output), nelem(input), threshold, val, state_stream(s)));
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaThreshold_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput,
                                                            THCudaTensor *gradInput, float threshold, float, bool inplace)
{
    TH_CHECK(s, nelem(input) == nelem(gradOutput), "input and gradOutput have different number of elements");
    THCudaTensor *x = new_contiguous(s, input), *gy = new_contiguous(s, gradOutput);
    if (x && gy) {
        if (inplace) {
            if (gy != gradOutput) raise(s, "in-place Threshold needs a contiguous gradOutput");
            else TH_CALL(s, cunn_b200_threshold_backward(tdata<float>(x), tdata<float>(gy), tdata<float>(gy), nelem(input), threshold, state_stream(s)));
        } else if (tensor_resize(s, gradInput, input->nDimension, input->size, 4)) {
            TH_CALL(s, cunn_b200_threshold_backward(tdata<float>(x), tdata<float>(gy), tdata<float>(gradInput), nelem(input), threshold, state_stream(s)));
        }
    }
done:
    tensor_free(s, x); tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaSpatialAveragePooling_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output, int kW,
                                                                     int kH, int dW, int dH, int padW, int padH, bool ceil_mode,
                                                                     bool count_include_pad)
{
    const int nd = input->nDimension;
    TH_CHECK(s, nd == 3 || nd == 4, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str());
    TH_CHECK(s, kW > 0 && kH > 0 && dW > 0 && dH > 0, "kernel size and stride should be greater than zero");
    const int b = nd == 4;
    const long N = b ? input->size[0] : 1, C = input->size[b], H = input->size[b + 1], W = input->size[b + 2];
    const long oH = cunn_b200_maxpool_out_size((int)H, kH, dH, padH, 1, ceil_mode), oW = cunn_b200_maxpool_out_size((int)W, kW, dW, padW, 1, ceil_mode);
    TH_CHECK(s, oH >= 1 && oW >= 1, "Given input size: (%ldx%ldx%ld). Calculated output size: (%ldx%ldx%ld). Output size is too small", C, H, W, C, oH, oW);
    THCudaTensor *x = new_contiguous(s, input);
    const long sz4[4] = {N, C, oH, oW};
    if (x && tensor_resize(s, output, 4, sz4, 4)) {
        TH_CALL(s, cunn_b200_avgpool_forward(tdata<float>(x), tdata<float>(output), (int)N, (int)C, (int)H, (int)W, (int)oH, (int)oW, kH, kW, dH, dW,
                                             padH, padW, count_include_pad, state_stream(s)));
        if (nd == 3) tensor_resize(s, output, 3, sz4 + 1, 4);
    }
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaSpatialAveragePooling_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput,
                                                                        THCudaTensor *gradInput, int kW, int kH, int dW, int dH,
                                                                        int padW, int padH, bool ceil_mode, bool count_include_pad)
{
    const int nd = input->nDimension;
    TH_CHECK(s, nd == 3 || nd == 4, "3D or 4D input tensor expected but got: %s", size_desc(input).c_str());
    const int b = nd == 4;
    const long N = b ? input->size[0] : 1, C = input->size[b], H = input->size[b + 1], W = input->size[b + 2];
    const long oH = cunn_b200_maxpool_out_size((int)H, kH, dH, padH, 1, ceil_mode), oW = cunn_b200_maxpool_out_size((int)W, kW, dW, padW, 1, ceil_mode);
    TH_CHECK(s, gradOutput->nDimension == nd && gradOutput->size[b + 1] == oH && gradOutput->size[b + 2] == oW,
             "gradOutput has the wrong shape: %s", size_desc(gradOutput).c_str());
    THCudaTensor *gy = new_contiguous(s, gradOutput);
    if (gy && tensor_resize(s, gradInput, nd, input->size, 4))
        TH_CALL(s, cunn_b200_avgpool_backward(tdata<float>(gy), tdata<float>(gradInput), (int)N, (int)C, (int)H, (int)W, (int)oH, (int)oW, kH, kW, dH,
                                              dW, padH, padW, count_include_pad, state_stream(s)));
done:
    tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaLogSoftMax_updateOutput(THCState *s, THCudaTensor *input, THCudaTensor *output)
{
    TH_CHECK(s, input->nDimension == 1 || input->nDimension == 2, "vector or matrix expected");
    const long B = input->nDimension == 2 ? input->size[0] : 1, D = input->size[input->nDimension - 1];
    THCudaTensor *x = new_contiguous(s, input);
    if (x && tensor_resize(s, output, input->nDimension, input->size, 4))
        TH_CALL(s, cunn_b200_logsoftmax_forward(tdata<float>(x), tdata<float>(output), (int)B, (int)D, state_stream(s)));
done:
    tensor_free(s, x);
}

extern "C" CUNN_API void THNN_CudaLogSoftMax_updateGradInput(THCState *s, THCudaTensor *input, THCudaTensor *gradOutput,
                                                             THCudaTensor *gradInput, THCudaTensor *output)
{
    TH_CHECK(s, output->nDimension == 1 || output->nDimension == 2, "vector or matrix expected");
    TH_CHECK(s, nelem(output) == nelem(gradOutput), "output and gradOutput have different number of elements");
    const long B = output->nDimension == 2 ? output->size[0] : 1, D = output->size[output->nDimension - 1];
    THCudaTensor *y = new_contiguous(s, output), *gy = new_contiguous(s, gradOutput);
    if (y && gy && tensor_resize(s, gradInput, output->nDimension, output->size, 4))
        TH_CALL(s, cunn_b200_logsoftmax_backward(tdata<float>(y), tdata<float>(gy), tdata<float>(gradInput), (int)B, (int)D, state_stream(s)));
done:
    (void)input;
    tensor_free(s, y); tensor_free(s, gy);
}

extern "C" CUNN_API void THNN_CudaClassNLLCriterion_updateOutput(THCState *s, THCudaTensor *input, THCudaLongTensor *target,
                                                                 THCudaTensor *output, bool sizeAverage, THCudaTensor *weights,
                                                                 THCudaTensor *total_weight, long ignore_index)
{
    TH_CHECK(s, input->nDimension == 1 || input->nDimension == 2, "input tensor should be 1D or 2D");
    const long B = input->nDimension == 2 ? input->size[0] : 1, D = input->size[input->nDimension - 1];
    TH_CHECK(s, nelem(target) == B, "mismatch between the batch size of input (%ld) and that of target (%td)", B, nelem(target));
    TH_CHECK(s, !weights || nelem(weights) == D, "weight tensor should be defined either for all %ld classes or no classes", D);
    TH_CHECK(s, is_contiguous(input) && is_contiguous(target) && (!weights || is_contiguous(weights)), "input, target and weights have to be contiguous");
    const long one[1] = {1};
    if (!(tensor_resize(s, output, 1, one, 4) && tensor_resize(s, total_weight, 1, one, 4))) return;
    // the flat ABI writes loss and total weight side by side; route them through the state's scratch
    float *pair = (float *)state_scratch(s, 0, 16);
    if (!pair) return;
    if (cunn_b200_classnll_forward(tdata<float>(input), tdata<int64_t>(target), weights ? tdata<float>(weights) : nullptr, pair, (int)B, (int)D,
                                   sizeAverage, ignore_index, state_stream(s))) {
        raise(s, "%s", cunn_b200_last_error());
        return;
    }
    cudaMemcpyAsync(tdata<float>(output), pair, 4, cudaMemcpyDeviceToDevice, state_stream(s));
    cudaMemcpyAsync(tdata<float>(total_weight), pair + 1, 4, cudaMemcpyDeviceToDevice, state_stream(s));
}

extern "C" CUNN_API void THNN_CudaClassNLLCriterion_updateGradInput(THCState *s, THCudaTensor *input, THCudaLongTensor *target,
                                                                    THCudaTensor *gradInput, bool sizeAverage, THCudaTensor *weights,
                                                                    THCudaTensor *total_weight, long ignore_index)
{
    TH_CHECK(s, input->nDimension == 1 || input->nDimension == 2, "input tensor should be 1D or 2D");
    const long B = input->nDimension == 2 ? input->size[0] : 1, D = input->size[input->nDimension - 1];
    TH_CHECK(s, nelem(target) == B, "mismatch between the batch size of input (%ld) and that of target (%td)", B, nelem(target));
    // gradInput is NOT zeroed here: nn.ClassNLLCriterion resizes and zeroes it before the call
    TH_CHECK(s, nelem(gradInput) == nelem(input) && is_contiguous(gradInput), "gradInput must be contiguous and of input's size");
    if (cunn_b200_classnll_backward(tdata<int64_t>(target), weights ? tdata<float>(weights) : nullptr, tdata<float>(total_weight), tdata<float>(gradInput),
                                    (int)B, (int)D, sizeAverage, ignore_index, state_stream(s)))
        raise(s, "%s", cunn_b200_last_error());
}
