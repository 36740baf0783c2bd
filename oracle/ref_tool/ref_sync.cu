// TEST INFRASTRUCTURE.  The switch read by ref_finish() (ref_sync.h).
#include "ref_sync.h"
int g_ref_sync = 1;
extern "C" void ref_set_sync(int on) { g_ref_sync = on; }
