// Error text of the C interface.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

static thread_local char g_error[512] = "";

void mlxone_set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
}

// Text of the last error that a call on this thread reported.
MLXONE_API const char* mlxone_last_error() { return g_error; }

// Version of the C interface; the Python side checks it after loading the library.
MLXONE_API int mlxone_abi_version() { return 1; }

static bool g_pdl = true;
bool mlxone_pdl_enabled() { return g_pdl; }

// Turns programmatic dependent launches of the decode path on (1, the default) or off (0).
MLXONE_API void mlxone_set_pdl(int enabled) { g_pdl = enabled != 0; }
MLXONE_API int mlxone_get_pdl() { return g_pdl ? 1 : 0; }
