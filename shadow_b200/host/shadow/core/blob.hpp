// Same include path as the reference (shadow/core/blob.hpp); everything lives in shadow_api.hpp.
#include "../shadow_api.hpp"
