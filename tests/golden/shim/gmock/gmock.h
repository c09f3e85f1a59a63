// The reference's test_utils.h builds a vector of gmock float matchers in a
// helper none of the pinned tests call; these two names let it compile.
#ifndef GOLDEN_SHIM_GMOCK_H_
#define GOLDEN_SHIM_GMOCK_H_
#include "gtest/gtest.h"
namespace testing {
template <typename T> struct Matcher { T value; T tol; };
inline Matcher<float> FloatNear(float v, float tol) { return Matcher<float>{v, tol}; }
}  // namespace testing
#endif
