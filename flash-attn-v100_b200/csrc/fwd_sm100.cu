#include "fa_common.cuh"
namespace fa {
bool sm100_supports(const fa_b200_params& p, bool backward, const char** why) { *why = "not built yet"; return false; }
int sm100_fwd(const fa_b200_params& p) { return FA_EUNSUPPORTED; }
}
