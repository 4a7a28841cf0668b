/* Force-included in front of every reference translation unit built into oracle/_ref:
 * pulls in the standard headers the sources use, then turns their per-element printf
 * calls into no-ops so that the functions can be timed and called in bulk. */
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <iostream>
#include <string>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#define printf(...) ((void)0)
