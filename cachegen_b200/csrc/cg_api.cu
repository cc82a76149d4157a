// Version, status text and CUDA error capture of the C ABI.
#include "cg_common.cuh"

#include <string>

namespace cg {

static thread_local std::string g_last_error;

int set_cuda_error(cudaError_t e) {
    g_last_error = std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e);
    return CG_E_CUDA;
}

}  // namespace cg

extern "C" const char *cg_version(void) { return "cachegen_b200 0.1 (sm_100a)"; }

extern "C" const char *cg_last_cuda_error(void) { return cg::g_last_error.c_str(); }

extern "C" const char *cg_status_string(int code) {
    switch (code) {
        case CG_OK: return "ok";
        case CG_E_NULL: return "a required pointer is NULL";
        case CG_E_SHAPE: return "non-positive or inconsistent extent";
        case CG_E_TOKENS: return "more than 256 tokens in one coder call";
        case CG_E_LP: return "CDF length outside [2, 64] (max_bins outside [1, 63])";
        case CG_E_ALIGN: return "pointer or stride breaks an alignment rule of the call";
        case CG_E_CAPACITY: return "workspace too small or too many jobs";
        case CG_E_DTYPE: return "unknown 16-bit float type code";
        case CG_E_CUDA: return "the CUDA runtime refused the launch";
        case CG_E_HIST: return "65536 or more tokens in one table build";
        default: return "unknown status";
    }
}

extern "C" int cg_workspace_bytes(int nrows, int ntokens, int nchannels, cg_workspace_sizes *out_host) {
    if (!out_host) return CG_E_NULL;
    if (nrows <= 0 || ntokens <= 0 || nchannels <= 0) return CG_E_SHAPE;
    const int64_t nsub = (static_cast<int64_t>(ntokens) + CG_MAX_TOKENS_PER_STREAM - 1) / CG_MAX_TOKENS_PER_STREAM;
    const int64_t sub_tokens = ntokens < CG_MAX_TOKENS_PER_STREAM ? ntokens : CG_MAX_TOKENS_PER_STREAM;
    const int64_t stride = (CG_STREAM_CAPACITY(sub_tokens) + 3) / 4 * 4;
    const int64_t streams = static_cast<int64_t>(nrows) * nchannels;
    const int64_t groups = static_cast<int64_t>(nrows) * ((nchannels + CG_GROUP_CHANNELS - 1) / CG_GROUP_CHANNELS);
    out_host->nsub = nsub;
    out_host->scratch_stride = stride;
    out_host->encode_scratch = nsub * streams * stride;
    out_host->encode_lengths = nsub * streams * 4;
    out_host->encode_group_off = nsub * groups * 8;
    out_host->encode_sub_off = (nsub + 1) * 8;
    out_host->decode_group_off = groups * 8;
    out_host->symbols = streams * ntokens;
    return CG_OK;
}
