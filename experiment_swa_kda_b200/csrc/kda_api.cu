// C ABI for the chunked KDA operator: argument checks and lane dispatch.

#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "simt_ws.cuh"
#include "tc_ws.cuh"

namespace kda {
int simt_chunk_fwd(const KdaChunkShape* sh, const void* q, const void* k, const void* v, const void* g, const void* beta,
                   const float* h0, const int32_t* cu, void* o, float* final_state, void* workspace, cudaStream_t st,
                   const tc::NormEpilogue* norm, const tc::ConvPrep* conv = nullptr);
int chunk_status(const KdaChunkShape* sh, const void* workspace, cudaStream_t st);
int chunk_status_async(const KdaChunkShape* sh, const void* workspace, int32_t* host_word, cudaStream_t st);
int status_word_to_code(int v);
int simt_chunk_bwd(const KdaChunkShape* sh, const void* q, const void* k, const void* v, const void* g, const void* beta,
                   const int32_t* cu, const void* d_o, const float* d_final, const void* workspace, void* scratch,
                   void* dq, void* dk, void* dv, void* dg, void* dbeta, float* dh0, cudaStream_t st);
}  // namespace kda

using namespace kda;

static int check_shape(const KdaChunkShape* s, const int32_t* cu) {
    if (!s) return KDA_ERR_NULL;
    if (s->n_seq <= 0 || s->heads <= 0 || s->key_dim <= 0 || s->value_dim <= 0 || s->tokens < 0 || s->seq_len < 0)
        return KDA_ERR_BAD_SHAPE;
    if (s->key_dim > KDA_MAX_DIM || s->value_dim > KDA_MAX_DIM) return KDA_ERR_BAD_SHAPE;
    if (s->io_dtype != KDA_DTYPE_F32 && s->io_dtype != KDA_DTYPE_BF16) return KDA_ERR_UNSUPPORTED;
    if (s->gate_dtype != KDA_DTYPE_F32 && s->gate_dtype != KDA_DTYPE_BF16) return KDA_ERR_UNSUPPORTED;
    if (s->forward_only != 0 && s->forward_only != 1) return KDA_ERR_BAD_SHAPE;
    if (cu) {
        if (s->seq_len != 0) return KDA_ERR_BAD_SHAPE;   // packed batches describe lengths through cu_seqlens only
    } else {
        if ((long long)s->n_seq * s->seq_len != s->tokens) return KDA_ERR_BAD_SHAPE;
    }
    if (s->lane == KDA_LANE_TC) {
        // tensor-core tiles are built for 128-wide heads and bf16 activations
        if (s->key_dim != 128 || s->value_dim != 128 || s->io_dtype != KDA_DTYPE_BF16) return KDA_ERR_UNSUPPORTED;
    } else if (s->lane != KDA_LANE_FP32) {
        return KDA_ERR_UNSUPPORTED;
    }
    return KDA_OK;
}

extern "C" const char* kda_error_string(int code) {
    switch (code) {
        case KDA_OK: return "ok";
        case KDA_ERR_BAD_SHAPE: return "bad shape: a dimension is non-positive, above 256, or inconsistent with tokens / cu_seqlens";
        case KDA_ERR_UNSUPPORTED: return "unsupported lane, dtype or size for this entry point";
        case KDA_ERR_WORKSPACE: return "workspace or scratch buffer missing, misaligned or too small";
        case KDA_ERR_CUDA: return "CUDA runtime reported an error at launch";
        case KDA_ERR_NULL: return "required pointer is null";
        case KDA_ERR_DEVICE_STATUS: return "kernel reported a device-side status (bounded wait expired)";
        case KDA_ERR_CU_SEQLENS: return "cu_seqlens is inconsistent: not starting at 0, not ending at the token count, decreasing, or describing more chunks than the workspace holds";
        default: return "unknown error";
    }
}

extern "C" const char* kda_build_arch(void) { return "sm_100a"; }

extern "C" size_t kda_chunk_workspace_bytes(const KdaChunkShape* shape) {
    if (!shape || shape->n_seq <= 0 || shape->heads <= 0 || shape->key_dim <= 0 || shape->value_dim <= 0) return 0;
    size_t bytes = 0, tcb = 0;
    simt::carve_ws(*shape, nullptr, &bytes);
    if (shape->lane == KDA_LANE_TC) tc::carve_tc(*shape, nullptr, &tcb);
    return bytes + tcb;
}

extern "C" size_t kda_chunk_bwd_scratch_bytes(const KdaChunkShape* shape) {
    if (!shape || shape->n_seq <= 0 || shape->heads <= 0 || shape->key_dim <= 0 || shape->value_dim <= 0) return 0;
    size_t bytes = 0;
    simt::carve_scr(*shape, nullptr, &bytes);
    return bytes;
}

extern "C" int kda_chunk_fwd(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                             void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_shape(shape, cu_seqlens);
    if (rc) return rc;
    if (shape->tokens > 0 && (!q || !k || !v || !g || !beta || !o)) return KDA_ERR_NULL;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 256) != 0 ||
        workspace_bytes < kda_chunk_workspace_bytes(shape))
        return KDA_ERR_WORKSPACE;
    return simt_chunk_fwd(shape, q, k, v, g, beta, h0, cu_seqlens, o, final_state, workspace, (cudaStream_t)stream, nullptr);
}

extern "C" int kda_chunk_fwd_conv(const KdaChunkShape* shape, const void* xq, const void* xk, const void* xv, const void* wq,
                                  const void* wk, const void* wv, int32_t conv_width, int32_t weight_dtype, const void* g,
                                  const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_shape(shape, cu_seqlens);
    if (rc) return rc;
    // the convolution lives in the tensor-core lane's forward kernel, width 4 with SiLU, and only where nothing is kept for
    // a backward (which would need the activations in memory)
    if (shape->lane != KDA_LANE_TC || !shape->forward_only || conv_width != 4) return KDA_ERR_UNSUPPORTED;
    if (shape->tokens > 0 && (!xq || !xk || !xv || !wq || !wk || !wv || !g || !beta || !o)) return KDA_ERR_NULL;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 256) != 0 || workspace_bytes < kda_chunk_workspace_bytes(shape))
        return KDA_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(xk) | reinterpret_cast<uintptr_t>(xv) | reinterpret_cast<uintptr_t>(wq) |
         reinterpret_cast<uintptr_t>(wk) | reinterpret_cast<uintptr_t>(wv)) % 16 != 0)
        return KDA_ERR_UNSUPPORTED;
    tc::ConvPrep cp{{wq, wk, wv}, weight_dtype == KDA_DTYPE_F32 ? 1 : 0};
    return simt_chunk_fwd(shape, xq, xk, xv, g, beta, h0, cu_seqlens, o, final_state, workspace, (cudaStream_t)stream, nullptr, &cp);
}

extern "C" int kda_chunk_fwd_norm(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                                  const void* beta, const float* h0, const int32_t* cu_seqlens, void* o, float* final_state,
                                  void* workspace, size_t workspace_bytes, const void* gate, const float* norm_weight, float eps,
                                  void* y, float* inv_rms, void* stream) {
    int rc = check_shape(shape, cu_seqlens);
    if (rc) return rc;
    if (shape->lane != KDA_LANE_TC) return KDA_ERR_UNSUPPORTED;      // the epilogue lives in the tensor-core lane's output kernel
    if (shape->tokens > 0 && (!q || !k || !v || !g || !beta || !o || !gate || !norm_weight || !y || !inv_rms)) return KDA_ERR_NULL;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 256) != 0 || workspace_bytes < kda_chunk_workspace_bytes(shape))
        return KDA_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(norm_weight)) % 16 != 0)
        return KDA_ERR_UNSUPPORTED;
    tc::NormEpilogue ep{static_cast<const __nv_bfloat16*>(gate), norm_weight, eps, static_cast<__nv_bfloat16*>(y), inv_rms};
    return simt_chunk_fwd(shape, q, k, v, g, beta, h0, cu_seqlens, o, final_state, workspace, (cudaStream_t)stream, &ep);
}

extern "C" int kda_chunk_bwd(const KdaChunkShape* shape, const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const int32_t* cu_seqlens, const void* d_o, const float* d_final_state,
                             const void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
                             void* dq, void* dk, void* dv, void* dg, void* dbeta, float* dh0, void* stream) {
    int rc = check_shape(shape, cu_seqlens);
    if (rc) return rc;
    if (shape->forward_only) return KDA_ERR_UNSUPPORTED;      // that forward kept nothing for a backward
    if (shape->tokens > 0 && (!q || !k || !v || !g || !beta || !d_o || !dq || !dk || !dv || !dg || !dbeta))
        return KDA_ERR_NULL;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) % 256) != 0 ||
        workspace_bytes < kda_chunk_workspace_bytes(shape))
        return KDA_ERR_WORKSPACE;
    if (!scratch || (reinterpret_cast<uintptr_t>(scratch) % 256) != 0 ||
        scratch_bytes < kda_chunk_bwd_scratch_bytes(shape))
        return KDA_ERR_WORKSPACE;
    return simt_chunk_bwd(shape, q, k, v, g, beta, cu_seqlens, d_o, d_final_state, workspace, scratch, dq, dk, dv, dg,
                          dbeta, dh0, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// launch accounting
// ---------------------------------------------------------------------------------------------
namespace kda {
namespace prof {
namespace {
struct Rec {
    const char* name;
    cudaEvent_t a, b;
};
std::mutex mu;
bool enabled = false;
unsigned long long launches = 0;
std::vector<Rec> recs;
}  // namespace

void begin(const char* name, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(mu);
    ++launches;
    if (!enabled) return;
    Rec r{name, nullptr, nullptr};
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
    cudaEventRecord(r.a, st);
    recs.push_back(r);
}

void end(cudaStream_t st) {
    std::lock_guard<std::mutex> lk(mu);
    if (!enabled || recs.empty()) return;
    cudaEventRecord(recs.back().b, st);
}
}  // namespace prof
}  // namespace kda

extern "C" int kda_chunk_status(const KdaChunkShape* shape, const void* workspace, void* stream) {
    if (!shape || !workspace) return KDA_ERR_NULL;
    return chunk_status(shape, workspace, (cudaStream_t)stream);
}

extern "C" int kda_chunk_status_async(const KdaChunkShape* shape, const void* workspace, int32_t* host_word, void* stream) {
    if (!shape || !workspace || !host_word) return KDA_ERR_NULL;
    return chunk_status_async(shape, workspace, host_word, (cudaStream_t)stream);
}

extern "C" int kda_status_word_code(int32_t word) { return status_word_to_code(word); }

extern "C" unsigned long long kda_launch_count(void) {
    std::lock_guard<std::mutex> lk(kda::prof::mu);
    return kda::prof::launches;
}

extern "C" void kda_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(kda::prof::mu);
    kda::prof::enabled = on != 0;
}

extern "C" int kda_profile_report(char* out, size_t cap) {
    using namespace kda::prof;
    std::lock_guard<std::mutex> lk(mu);
    std::map<std::string, std::pair<int, double>> agg;
    for (auto& r : recs) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            auto& e = agg[r.name];
            e.first += 1;
            e.second += ms;
        }
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    recs.clear();
    std::string text;
    char line[256];
    for (auto& kv : agg) {
        snprintf(line, sizeof line, "%s,%d,%.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        text += line;
    }
    if (!out || cap == 0) return (int)text.size();
    size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
    memcpy(out, text.data(), n);
    out[n] = 0;
    return (int)n;
}
