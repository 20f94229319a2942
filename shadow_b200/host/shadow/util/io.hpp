// Same include path as the reference (shadow/util/io.hpp): IO::ReadProtoFromText / ReadProtoFromTextFile.
#include "../shadow_api.hpp"
