// Host-side helpers shared by the translation units of libfeather_b200: the thread-local error text
// behind feather_last_error_string().
#pragma once
#include <stdarg.h>
#include <stdio.h>

namespace feather {

char* error_buffer();   // 512 bytes, thread-local (defined in quant.cu)

inline int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace feather
