// TEST INFRASTRUCTURE.  How a launch shim ends: by default it waits for the device and
// returns the error state (what the fixture generator wants); with ref_set_sync(0) it
// returns at once, so that a timing harness can bracket several launches with CUDA events
// without host round trips in between.
#pragma once
#include <cuda_runtime.h>
extern int g_ref_sync;
static inline int ref_finish() { return g_ref_sync ? (int)cudaDeviceSynchronize() : (int)cudaGetLastError(); }
