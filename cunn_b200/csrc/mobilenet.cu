// MobileNetV1 training step built only from this library's C ABI entry points: the replica body that a
// batch-sharded DataParallelTable runs on each GPU.
//
//   stem  SpatialConvolutionMM 3x3 s2 p1 (3 -> 32) + BN + ReLU
//   13 x  [SpatialDepthWiseConvolution 3x3 p1 (stride 1|2) + BN + ReLU,
//          SpatialConvolutionMM 1x1 + BN + ReLU]
//   SpatialAveragePooling (global) -> Linear -> LogSoftMax -> ClassNLLCriterion
//
// Parameters live in ONE flat buffer in module order (weight, bias, BN gamma, BN beta per convolution,
// then the classifier), gradients in a second flat buffer of the same layout that the kernels
// accumulate into directly: that is the buffer the data-parallel step all-reduces.  BN running
// statistics are per-replica buffers and are never reduced (DataParallelTable.lua:247-265 reduces
// parameters only).  The library allocates nothing: activations and scratch come from a caller-owned arena.
#include "common.cuh"

#include <vector>
#include <algorithm>

namespace cunn {
namespace net {

enum Kind : int { KIND_STEM = 0, KIND_DW = 1, KIND_PW = 2 };

struct Layer {
    int kind, cin, cout, stride, hin, hout;
    long long w_off, b_off, g_off, beta_off;   // offsets in the flat parameter buffer (floats)
    long long bn_off;                          // running mean at bn_off, running var at bn_off + cout
    long long wcount;
};

struct Model {
    std::vector<Layer> layers;
    int feat = 0, classes = 0, final_hw = 0;
    long long fc_w_off = 0, fc_b_off = 0, nparams = 0, nbn = 0;
};

static int conv_out(int h, int k, int s, int p) { return (h + 2 * p - k) / s + 1; }

static bool build(const cunn_b200_mobilenet_config *cfg, Model &m)
{
    if (!cfg || cfg->image_hw < 32 || cfg->width_div < 1 || cfg->num_classes < 1 || 32 % cfg->width_div) return false;
    static const int chans[14] = {32, 64, 128, 128, 256, 256, 512, 512, 512, 512, 512, 512, 1024, 1024};
    static const int strides[13] = {1, 2, 1, 2, 1, 2, 1, 1, 1, 1, 1, 2, 1};
    const int div = cfg->width_div;
    long long off = 0, bn = 0;
    int h = cfg->image_hw;
    auto add = [&](int kind, int cin, int cout, int stride, int k, int pad) {
        Layer L{};
        L.kind = kind; L.cin = cin; L.cout = cout; L.stride = stride; L.hin = h;
        L.hout = conv_out(h, k, stride, pad);
        L.wcount = (kind == KIND_DW) ? (long long)cout * k * k : (long long)cout * cin * k * k;
        L.w_off = off; off += L.wcount;
        L.b_off = off; off += cout;
        L.g_off = off; off += cout;
        L.beta_off = off; off += cout;
        L.bn_off = bn; bn += 2 * cout;
        h = L.hout;
        m.layers.push_back(L);
    };
    add(KIND_STEM, 3, chans[0] / div, 2, 3, 1);
    for (int i = 0; i < 13; ++i) {
        add(KIND_DW, chans[i] / div, chans[i] / div, strides[i], 3, 1);
        add(KIND_PW, chans[i] / div, chans[i + 1] / div, 1, 1, 0);
    }
    if (h < 1) return false;
    m.feat = chans[13] / div;
    m.classes = cfg->num_classes;
    m.final_hw = h;
    m.fc_w_off = off; off += (long long)m.classes * m.feat;
    m.fc_b_off = off; off += m.classes;
    m.nparams = off;
    m.nbn = bn;
    return true;
}

static size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

// Arena layout (bytes from the base), computed identically by the size query and the step.
struct Arena {
    std::vector<size_t> conv_out, act, save;   // per layer: pre-BN output, post-ReLU output, save_mean|save_std
    size_t pooled = 0, logits = 0, logprob = 0, glogits = 0, gpooled = 0, loss2 = 0, gA = 0, gB = 0, work = 0, dwwork = 0, bnwork = 0, total = 0;
    size_t work_bytes = 0, dwwork_bytes = 0, bnwork_bytes = 0;   // dwwork / bnwork: scratch of the depthwise parameter gradient and of
                                               // batch normalisation, whose ticket counters must stay zero between calls, so nothing else may use them
};

static void plan(const Model &m, int B, Arena &a)
{
    size_t off = 0;
    size_t max_act = 0;
    size_t work = 1 << 20, dwwork = 1 << 20, bnwork = 1 << 20;
    for (const Layer &L : m.layers) {
        const size_t n = (size_t)B * L.cout * L.hout * L.hout * sizeof(float);
        a.conv_out.push_back(off); off = align_up(off + n);
        a.act.push_back(off); off = align_up(off + n);
        a.save.push_back(off); off = align_up(off + 2 * (size_t)L.cout * sizeof(float));
        max_act = std::max(max_act, n);
        max_act = std::max(max_act, (size_t)B * L.cin * L.hin * L.hin * sizeof(float));
        bnwork = std::max(bnwork, cunn_b200_batchnorm_workspace(B, L.cout));
        if (L.kind == KIND_DW)
            dwwork = std::max(dwwork, cunn_b200_dwconv_acc_grad_workspace(B, L.cin, L.hin, L.hin, 1, 3, 3, L.stride, L.stride, 1, 1));
        else if (L.kind == KIND_PW)
            work = std::max(work, cunn_b200_convmm_acc_grad_workspace(B, L.cin, L.hin, L.hin, L.cout, 1, 1, 1, 1, 0, 0));
        else
            work = std::max(work, cunn_b200_convmm_acc_grad_workspace(B, L.cin, L.hin, L.hin, L.cout, 3, 3, L.stride, L.stride, 1, 1));
    }
    work = std::max(work, cunn_b200_convmm_acc_grad_workspace(B, m.feat, 1, 1, m.classes, 1, 1, 1, 1, 0, 0));
    a.pooled = off; off = align_up(off + (size_t)B * m.feat * 4);
    a.logits = off; off = align_up(off + (size_t)B * m.classes * 4);
    a.logprob = off; off = align_up(off + (size_t)B * m.classes * 4);
    a.glogits = off; off = align_up(off + (size_t)B * m.classes * 4);
    a.gpooled = off; off = align_up(off + (size_t)B * m.feat * 4);
    a.loss2 = off; off = align_up(off + 16);
    a.gA = off; off = align_up(off + max_act);
    a.gB = off; off = align_up(off + max_act);
    a.work = off; a.work_bytes = align_up(work); off += a.work_bytes;
    a.dwwork = off; a.dwwork_bytes = align_up(dwwork); off += a.dwwork_bytes;
    a.bnwork = off; a.bnwork_bytes = align_up(bnwork); off += a.bnwork_bytes;
    a.total = off;
}

#define STEP(call)              \
    do {                        \
        if ((call) != 0) return 1; \
    } while (0)

}  // namespace net
}  // namespace cunn

using namespace cunn;
using namespace cunn::net;

extern "C" CUNN_API long long cunn_b200_mobilenet_param_count(const cunn_b200_mobilenet_config *cfg)
{
    Model m;
    return build(cfg, m) ? m.nparams : -1;
}

extern "C" CUNN_API long long cunn_b200_mobilenet_bn_stat_count(const cunn_b200_mobilenet_config *cfg)
{
    Model m;
    return build(cfg, m) ? m.nbn : -1;
}

extern "C" CUNN_API int cunn_b200_mobilenet_num_layers(const cunn_b200_mobilenet_config *cfg)
{
    Model m;
    return build(cfg, m) ? (int)m.layers.size() : -1;
}

// info[0..11] = kind, cin, cout, stride, hin, hout, weight offset, bias offset, gamma offset, beta offset,
// running-stat offset, weight count.  layer == num_layers describes the classifier: kind = 3, cin = features,
// cout = classes, hin = final map size, weight / bias offsets.
extern "C" CUNN_API int cunn_b200_mobilenet_layer_info(const cunn_b200_mobilenet_config *cfg, int layer, long long *info)
{
    clear_error();
    Model m;
    CUNN_CHECK_ARG(build(cfg, m) && info, "bad MobileNet configuration");
    CUNN_CHECK_ARG(layer >= 0 && layer <= (int)m.layers.size(), "layer index out of range");
    if (layer == (int)m.layers.size()) {
        const long long v[12] = {3, m.feat, m.classes, 1, m.final_hw, 1, m.fc_w_off, m.fc_b_off, -1, -1, -1,
                                 (long long)m.classes * m.feat};
        for (int i = 0; i < 12; ++i) info[i] = v[i];
        return 0;
    }
    const Layer &L = m.layers[layer];
    const long long v[12] = {L.kind, L.cin, L.cout, L.stride, L.hin, L.hout, L.w_off, L.b_off, L.g_off, L.beta_off, L.bn_off, L.wcount};
    for (int i = 0; i < 12; ++i) info[i] = v[i];
    return 0;
}

extern "C" CUNN_API size_t cunn_b200_mobilenet_arena_bytes(const cunn_b200_mobilenet_config *cfg, int batch)
{
    Model m;
    if (!build(cfg, m) || batch <= 0) return 0;
    Arena a;
    plan(m, batch, a);
    return a.total;
}

extern "C" CUNN_API int cunn_b200_mobilenet_step(const cunn_b200_mobilenet_config *cfg, const float *images,
                                                 const int64_t *labels, int batch, float inv_global_batch,
                                                 const float *params, float *grads, float *bn_running, void *arena,
                                                 size_t arena_bytes, float *loss, double momentum, double eps,
                                                 cunn_stream_t stream)
{
    clear_error();
    Model m;
    CUNN_CHECK_ARG(build(cfg, m), "bad MobileNet configuration");
    CUNN_CHECK_ARG(batch >= 0, "negative batch");
    if (batch == 0) return 0;   // a replica without rows takes no part in the step (DataParallelTable.lua:531)
    CUNN_CHECK_ARG(images && labels && params && grads && bn_running && arena && loss, "null pointer");
    Arena a;
    plan(m, batch, a);
    CUNN_CHECK_ARG(arena_bytes >= a.total && ((uintptr_t)arena & 255) == 0,
                   "MobileNet step needs an arena of %zu bytes aligned to 256, got %zu", a.total, arena_bytes);
    char *base = (char *)arena;
    auto F = [&](size_t off) { return (float *)(base + off); };
    void *work = base + a.work;
    const size_t wbytes = a.work_bytes;
    const int B = batch, nl = (int)m.layers.size();
    // the depthwise parameter-gradient kernel keeps ticket counters in the first 64 KiB of its workspace
    void *dwwork = base + a.dwwork;
    CUNN_CUDA(cudaMemsetAsync(dwwork, 0, 64 << 10, (cudaStream_t)stream));
    // batch normalisation keeps its ticket counters in the first 32 KiB of its own workspace
    void *bnwork = base + a.bnwork;
    const size_t bnbytes = a.bnwork_bytes;
    CUNN_CUDA(cudaMemsetAsync(bnwork, 0, cunn_b200_batchnorm_counter_bytes(), (cudaStream_t)stream));

    // ---------------- forward ----------------
    const float *x = images;
    for (int i = 0; i < nl; ++i) {
        const Layer &L = m.layers[i];
        float *co = F(a.conv_out[i]), *ac = F(a.act[i]), *sv = F(a.save[i]);
        const float *w = params + L.w_off, *b = params + L.b_off;
        if (L.kind == KIND_DW)
            STEP(cunn_b200_dwconv_forward(x, w, b, co, B, L.cin, L.hin, L.hin, 1, 3, 3, L.stride, L.stride, 1, 1, stream));
        else if (L.kind == KIND_PW)
            STEP(cunn_b200_convmm_forward(x, w, b, co, B, L.cin, L.hin, L.hin, L.cout, 1, 1, 1, 1, 0, 0, stream));
        else
            STEP(cunn_b200_convmm_forward(x, w, b, co, B, L.cin, L.hin, L.hin, L.cout, 3, 3, L.stride, L.stride, 1, 1, stream));
        // BN + ReLU in one pass (the caller-side fusion of nn.SpatialBatchNormalization + nn.ReLU)
        STEP(cunn_b200_batchnorm_relu_forward(co, ac, params + L.g_off, params + L.beta_off, bn_running + L.bn_off,
                                              bn_running + L.bn_off + L.cout, sv, sv + L.cout, B, L.cout, L.hout * L.hout,
                                              1, momentum, eps, bnwork, bnbytes, stream));
        x = ac;
    }
    const int fh = m.final_hw;
    STEP(cunn_b200_avgpool_forward(x, F(a.pooled), B, m.feat, fh, fh, 1, 1, fh, fh, 1, 1, 0, 0, 1, stream));
    STEP(cunn_b200_convmm_forward(F(a.pooled), params + m.fc_w_off, params + m.fc_b_off, F(a.logits), B, m.feat, 1, 1,
                                  m.classes, 1, 1, 1, 1, 0, 0, stream));
    STEP(cunn_b200_logsoftmax_forward(F(a.logits), F(a.logprob), B, m.classes, stream));
    // loss: sum over the local rows of -logprob[target], scaled by 1 / global batch, so that the replicas'
    // losses add up to the global mean
    STEP(cunn_b200_classnll_forward(F(a.logprob), labels, nullptr, F(a.loss2), B, m.classes, 0, -100, stream));
    CUNN_CUDA(cudaMemsetAsync(loss, 0, sizeof(float), (cudaStream_t)stream));
    STEP(cunn_b200_sgd_update(loss, F(a.loss2), 1, -inv_global_batch, stream));   // loss = 0 + inv * sum

    // ---------------- backward ----------------
    CUNN_CUDA(cudaMemsetAsync(F(a.glogits), 0, (size_t)B * m.classes * 4, (cudaStream_t)stream));
    STEP(cunn_b200_fill(F(a.loss2) + 1, 1, 1.f / inv_global_batch, stream));    // "total weight" = global batch
    STEP(cunn_b200_classnll_backward(labels, nullptr, F(a.loss2) + 1, F(a.glogits), B, m.classes, 1, -100, stream));
    STEP(cunn_b200_logsoftmax_backward(F(a.logprob), F(a.glogits), F(a.glogits), B, m.classes, stream));
    STEP(cunn_b200_convmm_acc_grad(F(a.pooled), F(a.glogits), grads + m.fc_w_off, grads + m.fc_b_off, B, m.feat, 1, 1,
                                   m.classes, 1, 1, 1, 1, 0, 0, 1.f, work, wbytes, stream));
    STEP(cunn_b200_convmm_grad_input(F(a.glogits), params + m.fc_w_off, F(a.gpooled), B, m.feat, 1, 1, m.classes, 1, 1, 1,
                                     1, 0, 0, stream));
    float *g = F(a.gA), *g2 = F(a.gB);
    STEP(cunn_b200_avgpool_backward(F(a.gpooled), g, B, m.feat, fh, fh, 1, 1, fh, fh, 1, 1, 0, 0, 1, stream));
    for (int i = nl - 1; i >= 0; --i) {
        const Layer &L = m.layers[i];
        float *co = F(a.conv_out[i]), *sv = F(a.save[i]);
        const float *xin = (i == 0) ? images : F(a.act[i - 1]);
        STEP(cunn_b200_batchnorm_relu_backward(co, g, g2, grads + L.g_off, grads + L.beta_off, params + L.g_off,
                                               params + L.beta_off, bn_running + L.bn_off, bn_running + L.bn_off + L.cout, sv, sv + L.cout, B,
                                               L.cout, L.hout * L.hout, 1, 1.0, eps, bnwork, bnbytes, stream));
        // g2 = gradient w.r.t. the convolution output
        if (L.kind == KIND_DW) {
            STEP(cunn_b200_dwconv_acc_grad(xin, g2, grads + L.w_off, grads + L.b_off, B, L.cin, L.hin, L.hin, 1, 3, 3,
                                           L.stride, L.stride, 1, 1, 1.f, dwwork, a.dwwork_bytes, stream));
            STEP(cunn_b200_dwconv_grad_input(g2, params + L.w_off, g, B, L.cin, L.hin, L.hin, 1, 3, 3, L.stride, L.stride, 1,
                                             1, stream));
        } else {
            const int k = (L.kind == KIND_PW) ? 1 : 3, pad = (L.kind == KIND_PW) ? 0 : 1;
            STEP(cunn_b200_convmm_acc_grad(xin, g2, grads + L.w_off, grads + L.b_off, B, L.cin, L.hin, L.hin, L.cout, k, k,
                                           L.stride, L.stride, pad, pad, 1.f, work, wbytes, stream));
            if (i > 0)   // the first layer has no input gradient
                STEP(cunn_b200_convmm_grad_input(g2, params + L.w_off, g, B, L.cin, L.hin, L.hin, L.cout, k, k, L.stride,
                                                 L.stride, pad, pad, stream));
        }
    }
    return 0;
}
