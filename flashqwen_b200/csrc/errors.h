// Error plumbing shared by the CUDA and host halves of libfqb: a per-thread message that
// fqb_last_error() returns. Nothing here exits or throws.
#pragma once

namespace fqb {

// Records a printf-style message for the calling thread and returns `code` unchanged.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

}  // namespace fqb
