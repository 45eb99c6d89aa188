// placeholder replaced below
#include "common.h"
namespace vb { int launch_gemm_tc(const GemmArgs&, bool* handled) { *handled = false; return VB_OK; } }
