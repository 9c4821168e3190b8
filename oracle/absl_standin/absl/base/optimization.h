// Minimal stand-in for the one Abseil macro the reference's CPU attention layer uses.
// Test infrastructure only: lets oracle/Makefile compile the reference sources in place.
#pragma once
#define ABSL_PREDICT_FALSE(x) (__builtin_expect(false || (x), false))
#define ABSL_PREDICT_TRUE(x) (__builtin_expect(false || (x), true))
