// placeholder until the tcgen05 forward lands
#include "qfa_common.cuh"
namespace qfa {
int attn_fwd_tc_supported(const QfaFwdArgs&) { return 0; }
int attn_fwd_tc_entry(const QfaFwdArgs&, cudaStream_t) { return QFA_ERR_MODE; }
}  // namespace qfa
