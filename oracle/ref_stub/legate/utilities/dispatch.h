// Stand-in for legate/utilities/dispatch.h: the tree task bodies include it but use only the
// reference's own type_dispatch helpers (cpp_utils.h); dim_dispatch lives in the main stand-in.
#pragma once
#include "legate.h"
