// Train-step driver for sequential conv/linear networks: the host-side op sequence of one
// Ferrox training step, issued through the library's own C-ABI entry points.
// It owns no device memory: parameters, gradients and the activation arena are bound by the
// caller (the pool stays the allocator).
#include "fxb_common.cuh"

#include <vector>

namespace fxb {

struct NetLayer {
    int kind, act;
    // input / output geometry
    int64_t in_c, in_h, in_w, out_c, out_h, out_w;
    int64_t k, stride, pad;
    int64_t w_off = -1, b_off = -1, end_off = -1;  // elements in the flat parameter buffer
    int64_t act_off = 0;                           // bytes in the arena: this layer's output
    // conv layers (f32): the layer input packed for the filter-gradient kernel, written by the forward
    // pass and read by the backward pass of the same step
    size_t packed_off = 0, packed_bytes = 0;
    int packed_valid = 0;
    // conv layers (f32) that follow a conv layer: this layer's input as class slabs, written by the epilogue of
    // the layer before it (its padding cells are zeroed once, at the first forward pass after a bind)
    size_t slab_off = 0, slab_bytes = 0;
    int slab_valid = 0;
    int param_index = -1;
    fxb_conv2d_desc cd{};
};

struct Net {
    Context* ctx;
    size_t es;
    int64_t batch;
    int64_t in_c, in_h, in_w;
    std::vector<NetLayer> layers;
    std::vector<int> param_layers;  // layer indices that own parameters
    int64_t nparams = 0;
    int64_t classes = 0;
    // arena layout (bytes)
    size_t arena_bytes = 0, g0_off = 0, g1_off = 0, ws_off = 0, ws_bytes = 0;
    // bound buffers
    char* params = nullptr;
    char* grads = nullptr;
    char* arena = nullptr;
    bool slabs_zeroed = false;
    // backward cursor
    int cur_grad = 0;  // which ping-pong buffer holds dL/d(output of the layer about to run)
};

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace fxb

using namespace fxb;

extern "C" size_t fxb_linear_bwd_workspace_bytes(fxb_handle_t, int64_t, int64_t, int64_t, size_t);
extern "C" size_t fxb_linear_fwd_workspace_bytes(fxb_handle_t, int64_t, int64_t, int64_t, size_t);
extern "C" size_t fxb_conv2d_wgrad_workspace_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);
extern "C" size_t fxb_conv2d_fprop_workspace_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);
extern "C" size_t fxb_conv2d_dgrad_workspace_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);
extern "C" size_t fxb_conv2d_backward_workspace_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);
extern "C" size_t fxb_conv2d_packed_input_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);
extern "C" size_t fxb_conv2d_input_slab_bytes(fxb_handle_t, const fxb_conv2d_desc*, size_t);

extern "C" int fxb_net_create(fxb_handle_t h, size_t elem_size, const fxb_layer_desc* layers, int nlayers, int64_t batch,
                              int64_t in_c, int64_t in_h, int64_t in_w, fxb_net_t* out) {
    Context* c = reinterpret_cast<Context*>(h);
    if (!c) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    FXB_CHECK_ARG(c, out != nullptr && layers != nullptr && nlayers > 0, "fxb_net_create: bad arguments");
    FXB_CHECK_ARG(c, elem_size == 4 || elem_size == 8, "fxb_net_create: element size must be 4 or 8");
    FXB_CHECK_ARG(c, batch > 0 && in_c > 0 && in_h > 0 && in_w > 0, "fxb_net_create: bad input shape");
    Net* n = new Net();
    n->ctx = c; n->es = elem_size; n->batch = batch; n->in_c = in_c; n->in_h = in_h; n->in_w = in_w;
    int64_t cc = in_c, hh = in_h, ww = in_w;
    size_t off = 0, max_act = (size_t)batch * in_c * in_h * in_w;
    size_t ws = 0;
    for (int i = 0; i < nlayers; ++i) {
        NetLayer L;
        L.kind = layers[i].kind; L.act = layers[i].act;
        L.in_c = cc; L.in_h = hh; L.in_w = ww;
        L.k = layers[i].kernel; L.stride = layers[i].stride; L.pad = layers[i].pad;
        if (L.kind == FXB_LAYER_CONV) {
            if (L.k <= 0 || L.stride <= 0 || L.pad < 0 || layers[i].out_channels <= 0 || hh + 2 * L.pad < L.k || ww + 2 * L.pad < L.k) {
                delete n;
                return fail(c, FXB_ERR_INVALID_ARGUMENT, "fxb_net_create: bad conv layer " + std::to_string(i));
            }
            L.out_c = layers[i].out_channels;
            L.out_h = (hh + 2 * L.pad - L.k) / L.stride + 1;
            L.out_w = (ww + 2 * L.pad - L.k) / L.stride + 1;
            L.cd = fxb_conv2d_desc{batch, cc, hh, ww, L.out_c, L.k, L.k, L.stride, L.stride, L.pad, L.pad};
            L.w_off = n->nparams; L.b_off = L.w_off + L.out_c * cc * L.k * L.k; L.end_off = L.b_off + L.out_c;
            ws = std::max(ws, fxb_conv2d_wgrad_workspace_bytes(h, &L.cd, elem_size));
            ws = std::max(ws, fxb_conv2d_fprop_workspace_bytes(h, &L.cd, elem_size));
            if (i > 0) {
                ws = std::max(ws, fxb_conv2d_backward_workspace_bytes(h, &L.cd, elem_size));
                L.packed_bytes = fxb_conv2d_packed_input_bytes(h, &L.cd, elem_size);
                if (n->layers.back().kind == FXB_LAYER_CONV) L.slab_bytes = fxb_conv2d_input_slab_bytes(h, &L.cd, elem_size);
            }
        } else if (L.kind == FXB_LAYER_LINEAR) {
            if (hh != 1 || ww != 1 || layers[i].out_channels <= 0) {
                delete n;
                return fail(c, FXB_ERR_INVALID_ARGUMENT, "fxb_net_create: linear layer " + std::to_string(i) + " needs a flattened input");
            }
            L.out_c = layers[i].out_channels; L.out_h = 1; L.out_w = 1;
            L.w_off = n->nparams; L.b_off = L.w_off + L.out_c * cc; L.end_off = L.b_off + L.out_c;
            ws = std::max(ws, fxb_linear_bwd_workspace_bytes(h, batch, cc, L.out_c, elem_size));
            ws = std::max(ws, fxb_linear_fwd_workspace_bytes(h, batch, cc, L.out_c, elem_size));
        } else if (L.kind == FXB_LAYER_FLATTEN) {
            L.out_c = cc * hh * ww; L.out_h = 1; L.out_w = 1;
        } else {
            delete n;
            return fail(c, FXB_ERR_INVALID_ARGUMENT, "fxb_net_create: unknown layer kind");
        }
        if (L.kind != FXB_LAYER_FLATTEN) {
            L.param_index = (int)n->param_layers.size();
            n->param_layers.push_back(i);
            n->nparams = L.end_off;
            L.act_off = off;
            const size_t elems = (size_t)batch * L.out_c * L.out_h * L.out_w;
            off += align256(elems * elem_size);
            max_act = std::max(max_act, elems);
            if (L.packed_bytes) {
                L.packed_off = off;
                off += align256(L.packed_bytes);
            }
            if (L.slab_bytes) {
                L.slab_off = off;
                off += align256(L.slab_bytes);
            }
        }
        cc = L.out_c; hh = L.out_h; ww = L.out_w;
        n->layers.push_back(L);
    }
    if (hh != 1 || ww != 1 || n->param_layers.empty() || n->layers.back().kind != FXB_LAYER_LINEAR) {
        delete n;
        return fail(c, FXB_ERR_INVALID_ARGUMENT, "fxb_net_create: the network must end in a linear layer producing [batch, classes]");
    }
    n->classes = cc;
    n->g0_off = off; off += align256(max_act * elem_size);
    n->g1_off = off; off += align256(max_act * elem_size);
    n->ws_off = off; n->ws_bytes = align256(ws); off += n->ws_bytes;
    n->arena_bytes = off;
    *out = reinterpret_cast<fxb_net_t>(n);
    return FXB_OK;
}

extern "C" int fxb_net_destroy(fxb_net_t net) {
    delete reinterpret_cast<Net*>(net);
    return FXB_OK;
}
extern "C" int64_t fxb_net_param_count(fxb_net_t net) { return net ? reinterpret_cast<Net*>(net)->nparams : 0; }
extern "C" int fxb_net_param_layers(fxb_net_t net) { return net ? (int)reinterpret_cast<Net*>(net)->param_layers.size() : 0; }
extern "C" size_t fxb_net_arena_bytes(fxb_net_t net) { return net ? reinterpret_cast<Net*>(net)->arena_bytes : 0; }
extern "C" int64_t fxb_net_num_classes(fxb_net_t net) { return net ? reinterpret_cast<Net*>(net)->classes : 0; }

extern "C" int fxb_net_param_offsets(fxb_net_t net, int i, int64_t* w, int64_t* b, int64_t* e) {
    Net* n = reinterpret_cast<Net*>(net);
    if (!n) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null network");
    FXB_CHECK_ARG(n->ctx, i >= 0 && i < (int)n->param_layers.size(), "fxb_net_param_offsets: layer index out of range");
    const NetLayer& L = n->layers[n->param_layers[i]];
    if (w) *w = L.w_off;
    if (b) *b = L.b_off;
    if (e) *e = L.end_off;
    return FXB_OK;
}

extern "C" int fxb_net_bind(fxb_net_t net, void* params, void* grads, void* arena, size_t arena_bytes) {
    Net* n = reinterpret_cast<Net*>(net);
    if (!n) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null network");
    FXB_CHECK_ARG(n->ctx, params && grads && arena, "fxb_net_bind: null buffer");
    if (arena_bytes < n->arena_bytes) return fail(n->ctx, FXB_ERR_WORKSPACE, "fxb_net_bind: arena smaller than fxb_net_arena_bytes");
    FXB_CHECK_ARG(n->ctx, (reinterpret_cast<uintptr_t>(arena) & 255) == 0, "fxb_net_bind: arena must be 256-byte aligned");
    n->params = static_cast<char*>(params); n->grads = static_cast<char*>(grads); n->arena = static_cast<char*>(arena);
    n->slabs_zeroed = false;
    return FXB_OK;
}

namespace {
template <typename T> struct Api;
template <> struct Api<float> {
    static int conv_fwd(fxb_handle_t h, const float* x, const float* w, const float* b, float* y, const fxb_conv2d_desc* d, int act,
                        void* ws, size_t wsb, void* packed, size_t packed_bytes, int* written, const void* in_slabs,
                        const fxb_conv2d_desc* next, void* out_slabs, size_t out_slab_bytes, int* out_written, fxb_stream_t st) {
        return fxb_conv2d_bias_act_fwd_chain_f32(h, x, w, b, y, d, act, ws, wsb, packed, packed_bytes, written, in_slabs, next,
                                                 out_slabs, out_slab_bytes, out_written, st);
    }
    static constexpr auto lin_fwd = fxb_linear_fwd_ws_f32;
    static constexpr auto lin_bwd = fxb_linear_bwd_f32;
    static constexpr auto conv_bwd = fxb_conv2d_backward_f32;
    static int ce(fxb_handle_t h, const void* z, const void* t, void* l, void* g, int64_t B, int64_t C, double s, fxb_stream_t st) {
        return fxb_softmax_ce_f32(h, (const float*)z, (const float*)t, (float*)l, (float*)g, B, C, (float)s, st);
    }
};
template <> struct Api<double> {
    static int conv_fwd(fxb_handle_t h, const double* x, const double* w, const double* b, double* y, const fxb_conv2d_desc* d,
                        int act, void* ws, size_t wsb, void*, size_t, int* written, const void*, const fxb_conv2d_desc*, void*,
                        size_t, int* out_written, fxb_stream_t st) {
        if (written) *written = 0;
        if (out_written) *out_written = 0;
        return fxb_conv2d_bias_act_fwd_f64(h, x, w, b, y, d, act, ws, wsb, st);
    }
    static constexpr auto lin_fwd = fxb_linear_fwd_ws_f64;
    static constexpr auto lin_bwd = fxb_linear_bwd_f64;
    static constexpr auto conv_bwd = fxb_conv2d_backward_f64;
    static int ce(fxb_handle_t h, const void* z, const void* t, void* l, void* g, int64_t B, int64_t C, double s, fxb_stream_t st) {
        return fxb_softmax_ce_f64(h, (const double*)z, (const double*)t, (double*)l, (double*)g, B, C, s, st);
    }
};

// Output buffer of layer li (flatten layers alias their producer); li == -1 is the network input.
const char* layer_output(const Net* n, int li, const void* x) {
    while (li >= 0 && n->layers[li].kind == FXB_LAYER_FLATTEN) --li;
    return li < 0 ? static_cast<const char*>(x) : n->arena + n->layers[li].act_off;
}

template <typename T>
int forward_t(Net* n, const void* x, fxb_stream_t st) {
    fxb_handle_t h = reinterpret_cast<fxb_handle_t>(n->ctx);
    if (!n->slabs_zeroed) {
        for (NetLayer& L : n->layers)
            if (L.slab_bytes) FXB_CUDA_OK(n->ctx, cudaMemsetAsync(n->arena + L.slab_off, 0, L.slab_bytes, static_cast<cudaStream_t>(st)));
        n->slabs_zeroed = true;
    }
    for (int i = 0; i < (int)n->layers.size(); ++i) {
        NetLayer& L = n->layers[i];
        if (L.kind == FXB_LAYER_FLATTEN) continue;
        const T* in = reinterpret_cast<const T*>(layer_output(n, i - 1, x));
        T* outp = reinterpret_cast<T*>(n->arena + L.act_off);
        const T* W = reinterpret_cast<const T*>(n->params) + L.w_off;
        const T* b = reinterpret_cast<const T*>(n->params) + L.b_off;
        int rc;
        void* ws = n->ws_bytes ? n->arena + n->ws_off : nullptr;
        if (L.kind == FXB_LAYER_CONV) {
            // the layer after this one, when it is a convolution that reads class slabs, gets them from this epilogue
            NetLayer* nx = (i + 1 < (int)n->layers.size() && n->layers[i + 1].slab_bytes) ? &n->layers[i + 1] : nullptr;
            if (nx) nx->slab_valid = 0;
            rc = Api<T>::conv_fwd(h, in, W, b, outp, &L.cd, L.act, ws, n->ws_bytes, L.packed_bytes ? n->arena + L.packed_off : nullptr,
                                  L.packed_bytes, &L.packed_valid, L.slab_valid ? n->arena + L.slab_off : nullptr,
                                  nx ? &nx->cd : nullptr, nx ? n->arena + nx->slab_off : nullptr, nx ? nx->slab_bytes : 0,
                                  nx ? &nx->slab_valid : nullptr, st);
        } else rc = Api<T>::lin_fwd(h, in, W, b, outp, n->batch, L.in_c, L.out_c, L.act, ws, n->ws_bytes, st);
        if (rc) return rc;
    }
    return FXB_OK;
}

template <typename T>
int backward_t(Net* n, const void* x, int last, int first, fxb_stream_t st) {
    fxb_handle_t h = reinterpret_cast<fxb_handle_t>(n->ctx);
    for (int pi = last; pi >= first; --pi) {
        const int li = n->param_layers[pi];
        const NetLayer& L = n->layers[li];
        const T* in = reinterpret_cast<const T*>(layer_output(n, li - 1, x));
        const T* outp = reinterpret_cast<const T*>(n->arena + L.act_off);
        const T* W = reinterpret_cast<const T*>(n->params) + L.w_off;
        T* dW = reinterpret_cast<T*>(n->grads) + L.w_off;
        T* db = reinterpret_cast<T*>(n->grads) + L.b_off;
        const T* dy = reinterpret_cast<const T*>(n->arena + (n->cur_grad ? n->g1_off : n->g0_off));
        T* dx = pi == 0 ? nullptr : reinterpret_cast<T*>(n->arena + (n->cur_grad ? n->g0_off : n->g1_off));
        void* ws = n->ws_bytes ? n->arena + n->ws_off : nullptr;
        const T* yact = L.act == FXB_ACT_NONE ? nullptr : outp;
        int rc;
        if (L.kind == FXB_LAYER_CONV) {
            rc = Api<T>::conv_bwd(h, in, dy, yact, W, dx, dW, db, &L.cd, L.act, ws, n->ws_bytes,
                                  L.packed_valid ? n->arena + L.packed_off : nullptr, st);
        } else {
            rc = Api<T>::lin_bwd(h, in, W, yact, dy, dx, dW, db, n->batch, L.in_c, L.out_c, L.act, ws, n->ws_bytes, st);
        }
        if (rc) return rc;
        if (dx) n->cur_grad ^= 1;
    }
    return FXB_OK;
}
}  // namespace

extern "C" int fxb_net_forward(fxb_net_t net, const void* x, void** logits_out, fxb_stream_t st) {
    Net* n = reinterpret_cast<Net*>(net);
    if (!n) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null network");
    FXB_CHECK_ARG(n->ctx, n->arena != nullptr, "fxb_net_forward: call fxb_net_bind first");
    FXB_CHECK_ARG(n->ctx, x != nullptr, "fxb_net_forward: null input");
    int rc = n->es == 4 ? forward_t<float>(n, x, st) : forward_t<double>(n, x, st);
    if (rc == FXB_OK && logits_out) *logits_out = n->arena + n->layers.back().act_off;
    return rc;
}

extern "C" int fxb_net_loss(fxb_net_t net, const void* targets, void* loss_out, double grad_scale, fxb_stream_t st) {
    Net* n = reinterpret_cast<Net*>(net);
    if (!n) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null network");
    FXB_CHECK_ARG(n->ctx, n->arena != nullptr && targets && loss_out, "fxb_net_loss: bad arguments");
    fxb_handle_t h = reinterpret_cast<fxb_handle_t>(n->ctx);
    const void* logits = n->arena + n->layers.back().act_off;
    n->cur_grad = 0;
    void* g = n->arena + n->g0_off;
    return n->es == 4 ? Api<float>::ce(h, logits, targets, loss_out, g, n->batch, n->classes, grad_scale, st)
                      : Api<double>::ce(h, logits, targets, loss_out, g, n->batch, n->classes, grad_scale, st);
}

extern "C" int fxb_net_backward_range(fxb_net_t net, const void* x, int last, int first, fxb_stream_t st) {
    Net* n = reinterpret_cast<Net*>(net);
    if (!n) return fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null network");
    FXB_CHECK_ARG(n->ctx, n->arena != nullptr && x != nullptr, "fxb_net_backward_range: bad arguments");
    FXB_CHECK_ARG(n->ctx, first >= 0 && last >= first && last < (int)n->param_layers.size(),
                  "fxb_net_backward_range: layer range out of bounds");
    return n->es == 4 ? backward_t<float>(n, x, last, first, st) : backward_t<double>(n, x, last, first, st);
}
