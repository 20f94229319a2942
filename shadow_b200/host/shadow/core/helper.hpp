// Same include path as the reference (shadow/core/helper.hpp); everything lives in shadow_api.hpp.
#include "../shadow_api.hpp"
