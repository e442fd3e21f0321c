#pragma once
#include <cstdarg>
#include <cstdio>
// gaspi_printf of GPI-2 goes to a logger daemon; here it is printf
inline void gaspi_printf(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vprintf(fmt, ap);
  va_end(ap);
}
