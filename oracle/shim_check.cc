// TEST INFRASTRUCTURE ONLY. Includes the FlashQwen tree's own declaration of the attention
// launchers (engine/src/attn_cute.h, found through the include path oracle/Makefile gives) and
// takes their addresses; the result links against libfqb.so with no undefined symbol allowed, which
// shows that the library's definitions have exactly the engine's signatures.
#include "attn_cute.h"

extern "C" {
void* shim_check_prefill() { return reinterpret_cast<void*>(&fq::LaunchAttnPrefillCute); }
void* shim_check_decode() { return reinterpret_cast<void*>(&fq::LaunchAttnDecodeCute); }
}
