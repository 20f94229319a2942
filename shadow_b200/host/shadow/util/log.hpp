// Same include path as the reference (shadow/util/log.hpp); everything lives in shadow_api.hpp.
#include "../shadow_api.hpp"
