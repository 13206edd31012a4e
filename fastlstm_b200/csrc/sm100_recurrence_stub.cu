#include "sm100.cuh"
namespace blstm {
bool sm100_recurrence_supported(const blstm_desc&, int) { return false; }
size_t sm100_recurrence_workspace(const blstm_desc&, int) { return 0; }
int sm100_fwd_recurrence(const blstm_desc&, void*, const void*, void*, void*, void*, size_t, cudaStream_t) { return BLSTM_E_UNSUPPORTED; }
int sm100_bwd_recurrence(const blstm_desc&, const void*, const void*, const void*, const void*, const void*, const void*, void*, void*, void*, float*, void*, size_t, cudaStream_t) { return BLSTM_E_UNSUPPORTED; }
}
