// Runs the reference's own in-binary known-answer suite (cuda/ctensortest.cu.h,
// CTensorTest<float>::Test) against the reference CPU backend (-DUSE_CPU forwards every
// cuda/*.cu.h header to cpu/*.h).  Exit code 0 = every reference known-answer check passed.
// Test infrastructure only; built by oracle/build.py into oracle/_ref/ref_selftest.
#include <cstring>
#include <string>
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cmath>

#include "cuda/ctensortest.cu.h"

int main()
{
    try {
        bool ok = CTensorTest<float>::Test();
        std::printf("\nreference CTensorTest<float>::Test() on the CPU backend: %s\n", ok ? "PASS" : "FAIL");
        return ok ? 0 : 1;
    } catch (const char *msg) {
        std::printf("reference threw: %s\n", msg);
        return 2;
    }
}
