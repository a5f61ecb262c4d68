// One decoder layer in one call from the host: the pre-norm arrangement with attention
// and a gated feed-forward, for the step function's eager steps.
//
// The parts of a layer are Python objects that each launch their kernels; a step of a
// few hundred launches then costs the host more than the device (a prompt portion of 512
// tokens on a 16-layer, 2,048-wide model: 3.4 ms of host time for 2.5 ms of kernels).
// This file is the same sequence of the same entry points, launched from C++ with what
// the parts decided for the step handed over in two structs: nothing here chooses a
// kernel, a split count or a route. The block part (parts/block.py) uses it when its
// norm, mixer and feed-forward are the standard ones in bfloat16 and falls back to its
// own calls for every other combination, so toy parts and other arrangements are
// untouched. Library matrix products go to cuBLAS directly (the library torch has
// loaded already, found with dlopen; its handle works in a workspace the caller gives, so
// that it allocates nothing while a stream is being captured).
//
// The reference runs its layers from C++ as well
// (pulsarlm-core/src/engine/model/llama.cpp:61-94).
#include <dlfcn.h>

#include "common.cuh"

// ---- the entry points this file strings together (defined in the other sources)
struct PlDecodeRope {
    const void* k_new;
    const void* v_new;
    const double* inv_freq;
    int rotary;
};
struct PlPrefillMass;
PL_API int pl_add_rmsnorm(float* x, const void* delta, const void* weight, int weight_dtype, void* out,
                          const int32_t* rows, int n_rows, int hidden, float eps, int dtype, cudaStream_t stream);
PL_API int pl_swiglu(const void* in, void* out, int n_tokens, int width, int dtype, cudaStream_t stream);
PL_API int pl_gemm_bf16_skinny(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw,
                               int64_t ldy, int out_f32, int32_t* status, cudaStream_t stream);
PL_API int pl_gemm_bf16_skinny_gated_in(const void* gated, const void* w, void* y, int t, int n, int k,
                                        int64_t ld_gated, int64_t ldw, int64_t ldy, int out_f32, int32_t* status,
                                        cudaStream_t stream);
PL_API int pl_gemm_bf16_pair(const void* x, const void* w, void* y, int t, int n, int k, int64_t ldx, int64_t ldw,
                             int64_t ldy, int out_f32, int gated, int32_t* status, cudaStream_t stream);
PL_API int pl_rope_kv_write(void* q, const void* k, const void* v, int64_t row_stride, const int32_t* pos,
                            const int32_t* entry, const int32_t* table, int table_width, void* k_pool,
                            void* v_pool, int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                            const double* inv_freq, int rotary, int n_tokens, int n_heads, int n_kv_heads,
                            int head_dim, int dtype, const float* q_norm, const float* k_norm, float norm_eps,
                            int32_t* status, cudaStream_t stream);
PL_API int pl_attention_decode(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                               int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                               const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                               void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int n_splits, float* scratch,
                               const PlDecodeRope* rope, int32_t* status, cudaStream_t stream);
PL_API int pl_attention_decode_items(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                                     int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                                     const int32_t* table, int table_width, const int32_t* pos,
                                     const int32_t* entry, void* out, int64_t out_row_stride, int n_tokens,
                                     int n_heads, int n_kv_heads, int head_dim, int window, float scale,
                                     const int32_t* items, int n_items, const int32_t* token_slot, float* scratch,
                                     int32_t* counters, const PlDecodeRope* rope, int32_t* status,
                                     cudaStream_t stream);
PL_API int pl_attention_prefill_tcgen05(const void* q, int64_t q_row_stride, int n_tokens, const void* k_pool,
                                        const void* v_pool, int64_t page_stride, int64_t head_stride, int page_size,
                                        int n_pages, const int32_t* table, int table_width, const int32_t* tiles,
                                        int n_tiles, void* out, int64_t out_row_stride, int n_heads, int n_kv_heads,
                                        int head_dim, int window, float scale, int n_splits, float* scratch,
                                        int wide, const PlPrefillMass* mass, int32_t* status, cudaStream_t stream);

// One layer's tensors and constants (fixed when the weights are loaded). Matrices are
// bf16 [out, in]; the norm weights fp32 or bf16 by norm_dtype.
struct PlLayerWeights {
    const void* mixer_norm;
    const void* ff_norm;
    int norm_dtype;
    float eps;
    const void* qkv;      // [(n_heads + 2 n_kv_heads) head_dim, hidden]
    const void* o;        // [hidden, n_heads head_dim]
    const void* gate_up;  // [2 inter, hidden]
    const void* down;     // [hidden, inter]
    int hidden, n_heads, n_kv_heads, head_dim, inter;
    const double* inv_freq;  // [rotary / 2] or null
    int rotary;
    float scale;
    int window;
    void* k_pool;
    void* v_pool;
    int64_t page_stride, head_stride;
    int page_size, n_pages;
};

// Routes of a matrix product, as parts/linear.py names them.
// (PAIR_GATED: the gate/up product applies SwiGLU in its epilogue; SKINNY_GATED_IN: the down
// product forms silu(g) * u as it reads the gate/up product's output, no SwiGLU kernel.)
enum PlRoute : int {
    PL_ROUTE_LIBRARY = 0,
    PL_ROUTE_SKINNY = 1,
    PL_ROUTE_PAIR = 2,
    PL_ROUTE_PAIR_GATED = 3,
    PL_ROUTE_SKINNY_GATED_IN = 4
};

// One step's inputs, the parts' decisions for it, and its workspace (shared by the layers
// of equal shape, which run one after the other).
struct PlLayerStep {
    float* x;                // [T, hidden] residual stream
    const void* delta_in;    // bf16 [T, hidden] or null: added into x by the first norm
    void* delta_out;         // bf16 [T, hidden]: the feed-forward's output
    int n_tokens, n_decode;
    const int32_t* pos;
    const int32_t* entry;
    const int32_t* table;
    int table_width;
    int32_t* status;
    // workspace, all bf16
    void* h;         // [T, hidden]
    void* qkv;       // [T, (n_heads + 2 n_kv_heads) head_dim]
    void* attended;  // [T, n_heads head_dim]
    void* mixed;     // [T, hidden]
    void* gate_up;   // [T, 2 inter] (unused with the gated epilogue)
    void* act;       // [T, inter]
    int route_qkv, route_o, route_gate_up, route_down;
    // attention of the leading single tokens
    int fold_rope;             // 1: the decode kernel rotates q and stores the new keys itself
    const int32_t* items;      // work list, or null for equal shares
    int n_items;
    const int32_t* item_slots;
    int32_t* counters;
    int decode_splits;
    float* decode_scratch;
    // attention of the prompt portions behind them (tcgen05)
    const int32_t* tiles;
    int n_tiles, wide, prefill_splits;
    float* prefill_scratch;
    // library products
    void* library_workspace;
    int64_t library_workspace_bytes;
    // 1: in a step with both kinds of tokens the two attention kernels run side by side (the
    // single tokens' on a second stream, forked and joined with events): a prompt portion's
    // few tiles leave most SMs idle.
    int attention_side_by_side;
};

namespace {

// ---- cuBLAS, through the copy of the library that is already in the process
typedef int (*create_fn)(void**);
typedef int (*set_stream_fn)(void*, cudaStream_t);
typedef int (*set_workspace_fn)(void*, void*, size_t);
typedef int (*gemm_ex_fn)(void*, int, int, int, int, int, const void*, const void*, int, int, const void*, int, int,
                          const void*, void*, int, int, int, int);

struct Library {
    void* handle = nullptr;
    set_stream_fn set_stream = nullptr;
    set_workspace_fn set_workspace = nullptr;
    gemm_ex_fn gemm_ex = nullptr;
    int device = -1;
    bool failed = false;
};

int open_library(Library& lib) {
    int device = 0;
    cudaGetDevice(&device);
    if (lib.handle != nullptr && lib.device == device) {
        return 0;
    }
    if (lib.failed) {
        return pl_fail(3, "layer_forward: the matrix product library could not be opened before");
    }
    void* so = nullptr;
    for (const char* name : {"libcublas.so.12", "libcublas.so.13", "libcublas.so"}) {
        so = dlopen(name, RTLD_NOW | RTLD_NOLOAD);
        if (so == nullptr) {
            so = dlopen(name, RTLD_NOW);
        }
        if (so != nullptr) {
            break;
        }
    }
    if (so == nullptr) {
        lib.failed = true;
        return pl_fail(3, "layer_forward: libcublas not found: %s", dlerror());
    }
    create_fn create = reinterpret_cast<create_fn>(dlsym(so, "cublasCreate_v2"));
    lib.set_stream = reinterpret_cast<set_stream_fn>(dlsym(so, "cublasSetStream_v2"));
    lib.set_workspace = reinterpret_cast<set_workspace_fn>(dlsym(so, "cublasSetWorkspace_v2"));
    lib.gemm_ex = reinterpret_cast<gemm_ex_fn>(dlsym(so, "cublasGemmEx"));
    if (create == nullptr || lib.set_stream == nullptr || lib.set_workspace == nullptr || lib.gemm_ex == nullptr) {
        lib.failed = true;
        return pl_fail(3, "layer_forward: libcublas lacks an entry point this file calls");
    }
    void* handle = nullptr;
    if (create(&handle) != 0 || handle == nullptr) {
        lib.failed = true;
        return pl_fail(3, "layer_forward: cublasCreate failed");
    }
    lib.handle = handle;  // (one per process and device in use; lives until the process ends)
    lib.device = device;
    return 0;
}

// y[T, N] = x[T, K] w[N, K]^T in bf16 with fp32 accumulation. Column-major: y^T [N, T] =
// w (as [K, N] column-major, transposed) x^T ([K, T]).
int library_product(const PlLayerStep& s, const void* x, const void* w, void* y, int t, int n, int k,
                    cudaStream_t stream) {
    static Library lib;
    if (const int code = open_library(lib)) {
        return code;
    }
    PL_REQUIRE(s.library_workspace != nullptr && s.library_workspace_bytes >= (1 << 20),
               "layer_forward: a library product needs a workspace");
    const float one = 1.0f, zero = 0.0f;
    constexpr int kOpN = 0, kOpT = 1, kBf16 = 14 /* CUDA_R_16BF */, kCompute32F = 68, kDefaultTensorOp = 99;
    if (lib.set_stream(lib.handle, stream) != 0 ||
        lib.set_workspace(lib.handle, s.library_workspace, static_cast<size_t>(s.library_workspace_bytes)) != 0) {
        return pl_fail(3, "layer_forward: cuBLAS refused the stream or the workspace");
    }
    const int status = lib.gemm_ex(lib.handle, kOpT, kOpN, n, t, k, &one, w, kBf16, k, x, kBf16, k, &zero, y, kBf16, n,
                                   kCompute32F, kDefaultTensorOp);
    if (status != 0) {
        return pl_fail(3, "layer_forward: cublasGemmEx failed with status %d (t=%d n=%d k=%d)", status, t, n, k);
    }
    return 0;
}

// The second stream and the two events of the side-by-side attention (one set per process;
// the engine works on one device and one stream).
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    bool failed = false;
};

bool side_stream(SideStream& side) {
    if (side.stream != nullptr) {
        return true;
    }
    if (side.failed) {
        return false;
    }
    if (cudaStreamCreateWithFlags(&side.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&side.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&side.join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        side.failed = true;
        side.stream = nullptr;
        return false;
    }
    return true;
}

int product(const PlLayerStep& s, int route, const void* x, const void* w, void* y, int t, int n, int k,
            cudaStream_t stream) {
    switch (route) {
        case PL_ROUTE_SKINNY: return pl_gemm_bf16_skinny(x, w, y, t, n, k, k, k, n, 0, s.status, stream);
        case PL_ROUTE_PAIR: return pl_gemm_bf16_pair(x, w, y, t, n, k, k, k, n, 0, 0, s.status, stream);
        case PL_ROUTE_LIBRARY: return library_product(s, x, w, y, t, n, k, stream);
        default: return pl_fail(2, "layer_forward: unknown product route %d", route);
    }
}

}  // namespace

// x += delta_in; x += attention(norm(x)); delta_out = feed_forward(norm(x)) for one
// layer in bfloat16, with the kernels and settings the structs name.
PL_API int pl_layer_forward(const PlLayerWeights* w, const PlLayerStep* s, cudaStream_t stream) {
    PL_REQUIRE(w != nullptr && s != nullptr && s->n_tokens >= 1 && s->n_decode >= 0 && s->n_decode <= s->n_tokens,
               "layer_forward: bad arguments");
    const int t = s->n_tokens, hd = w->head_dim;
    const int q_width = w->n_heads * hd, kv_width = w->n_kv_heads * hd, qkv_width = q_width + 2 * kv_width;
    auto* qkv = static_cast<__nv_bfloat16*>(s->qkv);
    auto* attended = static_cast<__nv_bfloat16*>(s->attended);
    int code = pl_add_rmsnorm(s->x, s->delta_in, w->mixer_norm, w->norm_dtype, s->h, nullptr, t, w->hidden, w->eps,
                              PL_BF16, stream);
    if (code == 0) {
        code = product(*s, s->route_qkv, s->h, w->qkv, qkv, t, qkv_width, w->hidden, stream);
    }
    PlDecodeRope rope = {qkv + q_width, qkv + q_width + kv_width, w->inv_freq, w->rotary};
    const PlDecodeRope* fold = s->fold_rope ? &rope : nullptr;
    if (code == 0 && !s->fold_rope) {
        code = pl_rope_kv_write(qkv, qkv + q_width, qkv + q_width + kv_width, qkv_width, s->pos, s->entry, s->table,
                                s->table_width, w->k_pool, w->v_pool, w->page_stride, w->head_stride, w->page_size,
                                w->n_pages, w->inv_freq, w->rotary, t, w->n_heads, w->n_kv_heads, hd, PL_BF16, nullptr,
                                nullptr, 0.0f, s->status, stream);
    }
    // The single tokens' attention beside the prompt portions' when the step has both and is
    // not being captured: forked onto a second stream after what they both wait for, joined
    // before the o projection.
    static SideStream side;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    bool forked = false;
    cudaStream_t decode_stream = stream;
    if (code == 0 && s->attention_side_by_side && s->n_decode > 0 && s->n_decode < t &&
        cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone &&
        side_stream(side)) {
        if (cudaEventRecord(side.fork, stream) == cudaSuccess &&
            cudaStreamWaitEvent(side.stream, side.fork, 0) == cudaSuccess) {
            forked = true;
            decode_stream = side.stream;
        } else {
            cudaGetLastError();
        }
    }
    if (code == 0 && s->n_decode > 0) {
        if (s->items != nullptr) {
            code = pl_attention_decode_items(qkv, qkv_width, w->k_pool, w->v_pool, w->page_stride, w->head_stride,
                                             w->page_size, w->n_pages, s->table, s->table_width, s->pos, s->entry,
                                             attended, q_width, s->n_decode, w->n_heads, w->n_kv_heads, hd, w->window,
                                             w->scale, s->items, s->n_items, s->item_slots, s->decode_scratch,
                                             s->counters, fold, s->status, decode_stream);
        } else {
            code = pl_attention_decode(qkv, qkv_width, w->k_pool, w->v_pool, w->page_stride, w->head_stride,
                                       w->page_size, w->n_pages, s->table, s->table_width, s->pos, s->entry, attended,
                                       q_width, s->n_decode, w->n_heads, w->n_kv_heads, hd, w->window, w->scale,
                                       s->decode_splits, s->decode_scratch, fold, s->status, decode_stream);
        }
    }
    if (forked && cudaEventRecord(side.join, side.stream) != cudaSuccess) {
        return pl_fail(3, "layer_forward: cannot record the side stream's event: %s",
                       cudaGetErrorString(cudaGetLastError()));
    }
    if (code == 0 && s->n_decode < t) {
        PL_REQUIRE(s->tiles != nullptr && s->n_tiles > 0, "layer_forward: prompt portions need their tile list");
        code = pl_attention_prefill_tcgen05(qkv, qkv_width, t, w->k_pool, w->v_pool, w->page_stride, w->head_stride,
                                            w->page_size, w->n_pages, s->table, s->table_width, s->tiles, s->n_tiles,
                                            attended, q_width, w->n_heads, w->n_kv_heads, hd, w->window, w->scale,
                                            s->prefill_splits, s->prefill_scratch, s->wide, nullptr, s->status, stream);
    }
    if (forked && cudaStreamWaitEvent(stream, side.join, 0) != cudaSuccess) {
        return pl_fail(3, "layer_forward: cannot join the side stream: %s", cudaGetErrorString(cudaGetLastError()));
    }
    if (code == 0) {
        code = product(*s, s->route_o, attended, w->o, s->mixed, t, w->hidden, q_width, stream);
    }
    if (code == 0) {
        code = pl_add_rmsnorm(s->x, s->mixed, w->ff_norm, w->norm_dtype, s->h, nullptr, t, w->hidden, w->eps, PL_BF16,
                              stream);
    }
    if (code == 0) {
        if (s->route_gate_up == PL_ROUTE_PAIR_GATED) {
            code = pl_gemm_bf16_pair(s->h, w->gate_up, s->act, t, w->inter, w->hidden, w->hidden, w->hidden, w->inter, 0,
                                     1, s->status, stream);
        } else {
            code = product(*s, s->route_gate_up, s->h, w->gate_up, s->gate_up, t, 2 * w->inter, w->hidden, stream);
            if (code == 0 && s->route_down != PL_ROUTE_SKINNY_GATED_IN) {
                code = pl_swiglu(s->gate_up, s->act, t, w->inter, PL_BF16, stream);
            }
        }
    }
    if (code == 0 && s->route_down == PL_ROUTE_SKINNY_GATED_IN) {
        code = pl_gemm_bf16_skinny_gated_in(s->gate_up, w->down, s->delta_out, t, w->hidden, w->inter, 2 * w->inter,
                                            w->inter, w->hidden, 0, s->status, stream);
    } else if (code == 0) {
        code = product(*s, s->route_down, s->act, w->down, s->delta_out, t, w->hidden, w->inter, stream);
    }
    return code;
}
