// TEST INFRASTRUCTURE -- a stand-in for the few GoogleTest names the reference project's layer
// tests use, so that those test files can be compiled for the scalar specifications they define
// (class AttentionReference, class DeltaReference, Reference(...)) without GoogleTest, which this
// machine does not have.  Test bodies compile but are never registered or run: TEST / TEST_F
// declare ordinary functions nobody calls, and the assertion macros evaluate to a stream sink.
#ifndef PLUTO_ORACLE_GTEST_STANDIN_H_
#define PLUTO_ORACLE_GTEST_STANDIN_H_

namespace testing {

class Test {
 public:
  virtual ~Test() = default;

 protected:
  virtual void SetUp() {}
  virtual void TearDown() {}
};

namespace standin {
struct Sink {
  template <typename T>
  Sink& operator<<(const T&) { return *this; }
};
struct Void {
  void operator&(const Sink&) const {}
};
template <typename A, typename B>
bool Near(const A& a, const B& b, double tolerance) {
  const double d = static_cast<double>(a) - static_cast<double>(b);
  return (d < 0 ? -d : d) <= tolerance;
}
}  // namespace standin
}  // namespace testing

#define TEST(suite, name) [[maybe_unused]] static void suite##_##name##_TestBody()
#define TEST_F(fixture, name)                              \
  struct fixture##_##name##_Test : public fixture {        \
    void TestBody();                                       \
  };                                                       \
  void fixture##_##name##_Test::TestBody()

#define PLUTO_STANDIN_EXPECT_(condition) \
  if (static_cast<bool>(condition))      \
    ;                                    \
  else                                   \
    ::testing::standin::Sink()
#define PLUTO_STANDIN_ASSERT_(condition) \
  if (static_cast<bool>(condition))      \
    ;                                    \
  else                                   \
    return ::testing::standin::Void() & ::testing::standin::Sink()

#define EXPECT_TRUE(c) PLUTO_STANDIN_EXPECT_(c)
#define EXPECT_FALSE(c) PLUTO_STANDIN_EXPECT_(!(c))
#define EXPECT_EQ(a, b) PLUTO_STANDIN_EXPECT_((a) == (b))
#define EXPECT_GT(a, b) PLUTO_STANDIN_EXPECT_((a) > (b))
#define EXPECT_NEAR(a, b, t) PLUTO_STANDIN_EXPECT_(::testing::standin::Near((a), (b), (t)))
#define EXPECT_FLOAT_EQ(a, b) PLUTO_STANDIN_EXPECT_(::testing::standin::Near((a), (b), 4e-7 * ((b) < 0 ? -(b) : (b))))
#define ASSERT_TRUE(c) PLUTO_STANDIN_ASSERT_(c)
#define ASSERT_EQ(a, b) PLUTO_STANDIN_ASSERT_((a) == (b))
#define SCOPED_TRACE(x) static_cast<void>(x)

#endif  // PLUTO_ORACLE_GTEST_STANDIN_H_
