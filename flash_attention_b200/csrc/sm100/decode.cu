#include "../fa_common.cuh"
namespace fa {
bool decode_eligible(const FaKvcacheArgs&) { return false; }
int decode_plan(const FaKvcacheArgs&, int) { return 1; }
int decode_run(const FaKvcacheArgs&, int, cudaStream_t) { return 1; }
}
