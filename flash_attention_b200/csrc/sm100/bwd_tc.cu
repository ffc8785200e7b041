#include "../fa_common.cuh"
namespace fa {
bool bwd_tc_eligible(const FaBwdArgs&) { return false; }
int bwd_tc_main(const FaBwdArgs&, cudaStream_t) { return 1; }
}
