#include "fa_common.cuh"
namespace fa {
int sm100_bwd(const fa_b200_params& p, const BwdWorkspace& ws) { return FA_EUNSUPPORTED; }
}
