// Error reporting shared by the translation units that define C-ABI entry points.
#pragma once

namespace dtb {

// Stores a printf-style message for dtb_last_error() on the calling host thread; returns `code`.
int set_error(int code, const char* fmt, ...);

// DTB_OK when the current device has compute capability 10.x, else DTB_ERR_DEVICE / DTB_ERR_CUDA
// (message stored).
int require_sm100();

}  // namespace dtb
