// A small test runner with the subset of the Google Test interface that primitiv's own tests
// use (TEST / TEST_F with per-suite SetUpTestCase / TearDownTestCase, EXPECT_* / ASSERT_* with
// streamed messages, testing::AssertionResult), so that the reference's test sources can be
// compiled where they lie, unmodified, against the B200 device.  Google Test itself is not in
// this environment; nothing here comes from it.  Header-only; one translation unit defines
// MINITEST_MAIN before including it to get the registry and main().
#ifndef MINITEST_GTEST_GTEST_H_
#define MINITEST_GTEST_GTEST_H_

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <functional>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace testing {

class AssertionResult {
 public:
  explicit AssertionResult(bool ok) : ok_(ok) {}
  AssertionResult(const AssertionResult &o) : ok_(o.ok_), msg_(o.msg_) {}
  explicit operator bool() const { return ok_; }
  std::string message() const { return msg_; }
  template <typename T>
  AssertionResult &operator<<(const T &v) {
    std::ostringstream os;
    os << v;
    msg_ += os.str();
    return *this;
  }

 private:
  bool ok_;
  std::string msg_;
};

inline AssertionResult AssertionSuccess() { return AssertionResult(true); }
inline AssertionResult AssertionFailure() { return AssertionResult(false); }

class Test {
 public:
  virtual ~Test() {}
  static void SetUpTestCase() {}
  static void TearDownTestCase() {}
  virtual void SetUp() {}
  virtual void TearDown() {}
  virtual void TestBody() = 0;
};

namespace internal {

struct Case {
  std::string suite, name;
  std::function<Test *()> make;
  void (*suite_up)();
  void (*suite_down)();
};

struct State {
  std::vector<Case> cases;
  int failures_in_test = 0;
};

State &state();

inline int add_case(const char *suite, const char *name, std::function<Test *()> make, void (*up)(),
                    void (*down)()) {
  state().cases.push_back(Case{suite, name, make, up, down});
  return 0;
}

// Collects the streamed message of a failed expectation and reports it when destroyed.
class Failure {
 public:
  Failure(const char *file, int line, const std::string &what) {
    os_ << file << ":" << line << ": Failure\n" << what << "\n";
  }
  ~Failure() {
    std::cerr << os_.str() << std::endl;
    ++state().failures_in_test;
  }
  template <typename T>
  Failure &operator<<(const T &v) {
    os_ << v;
    return *this;
  }

 private:
  std::ostringstream os_;
};

// `return Voidify() = failure << ...;` lets ASSERT_* leave a void function after streaming.
struct Voidify {
  void operator=(const Failure &) const {}
};

template <typename T>
inline std::string show(const T &v) {
  std::ostringstream os;
  os << v;
  return os.str();
}
inline std::string show(std::nullptr_t) { return "nullptr"; }

// A statement-scope variable for the macros below: `if (Holder h{}) {} else <uses h>`.
struct Holder {
  std::string text;
  int code = 0;
  explicit operator bool() const { return false; }
};

inline bool truth(const AssertionResult &r, std::string *why) {
  if (!r) *why = r.message();
  return static_cast<bool>(r);
}
inline bool truth(bool b, std::string *) { return b; }

template <typename A, typename B>
inline bool equal(const A &a, const B &b) { return a == b; }

inline bool float_eq_4ulp(float a, float b) {
  if (a == b) return true;
  std::int32_t ai, bi;
  std::memcpy(&ai, &a, 4);
  std::memcpy(&bi, &b, 4);
  if (ai < 0) ai = static_cast<std::int32_t>(0x80000000u) - ai;
  if (bi < 0) bi = static_cast<std::int32_t>(0x80000000u) - bi;
  const std::int64_t d = static_cast<std::int64_t>(ai) - bi;
  return (d < 0 ? -d : d) <= 4;
}

}  // namespace internal

inline void InitGoogleTest(int *, char **) {}

}  // namespace testing

#define MINITEST_FAIL_(what) ::testing::internal::Failure(__FILE__, __LINE__, what)
// `switch (0) case 0: default:` keeps an unbraced `if (...) EXPECT_x(...); else ...` of the caller unambiguous
#define MINITEST_NONFATAL_(cond, what) \
  switch (0) case 0: default: if (cond) {} else MINITEST_FAIL_(what)
#define MINITEST_FATAL_(cond, what) \
  switch (0) case 0: default: if (cond) {} else return ::testing::internal::Voidify() = MINITEST_FAIL_(what)

#define MINITEST_BOOL_(expr, want, label, MODE)                                             \
  switch (0) case 0: default: if (::testing::internal::Holder h__{}) {} else                \
    MODE(::testing::internal::truth((expr), &h__.text) == want,                             \
         std::string("Value of: " label "\n  Expected: ") + (want ? "true" : "false") +     \
             (h__.text.empty() ? std::string() : "\n" + h__.text))

#define EXPECT_TRUE(expr) MINITEST_BOOL_(expr, true, #expr, MINITEST_NONFATAL_)
#define EXPECT_FALSE(expr) MINITEST_BOOL_(expr, false, #expr, MINITEST_NONFATAL_)
#define ASSERT_TRUE(expr) MINITEST_BOOL_(expr, true, #expr, MINITEST_FATAL_)
#define ASSERT_FALSE(expr) MINITEST_BOOL_(expr, false, #expr, MINITEST_FATAL_)

#define MINITEST_CMP_(a, b, op, label, MODE)                                                \
  MODE((a)op(b), std::string("Expected: (" #a ") " label " (" #b ")"))
#define EXPECT_EQ(a, b)                                                                     \
  MINITEST_NONFATAL_(::testing::internal::equal((a), (b)), std::string("Expected equality of\n  " #a "\n  " #b))
#define ASSERT_EQ(a, b)                                                                     \
  MINITEST_FATAL_(::testing::internal::equal((a), (b)), std::string("Expected equality of\n  " #a "\n  " #b))
#define EXPECT_NE(a, b) MINITEST_CMP_(a, b, !=, "!=", MINITEST_NONFATAL_)
#define EXPECT_GE(a, b) MINITEST_CMP_(a, b, >=, ">=", MINITEST_NONFATAL_)
#define EXPECT_GT(a, b) MINITEST_CMP_(a, b, >, ">", MINITEST_NONFATAL_)
#define EXPECT_LE(a, b) MINITEST_CMP_(a, b, <=, "<=", MINITEST_NONFATAL_)
#define EXPECT_LT(a, b) MINITEST_CMP_(a, b, <, "<", MINITEST_NONFATAL_)
#define EXPECT_FLOAT_EQ(a, b)                                                               \
  MINITEST_NONFATAL_(::testing::internal::float_eq_4ulp((a), (b)), std::string("Expected (4 ULPs): " #a " == " #b))
#define EXPECT_NEAR(a, b, err)                                                              \
  MINITEST_NONFATAL_(std::fabs((a) - (b)) <= (err), std::string("Expected |" #a " - " #b "| <= " #err))

#define MINITEST_THROW_(stmt, type, MODE)                                                   \
  switch (0) case 0: default: if (::testing::internal::Holder h__{}) {} else                \
    if ((h__.code = [&]() -> int {                                                          \
           try { stmt; } catch (const type &) { return 1; } catch (...) { return 2; }       \
           return 0; }()) == 1) {} else                                                     \
      MODE(false, std::string("Expected: " #stmt " throws " #type "\n  Actual: ") +         \
                      (h__.code == 0 ? "it throws nothing" : "it throws a different type"))
#define EXPECT_THROW(stmt, type) MINITEST_THROW_(stmt, type, MINITEST_NONFATAL_)
#define ASSERT_THROW(stmt, type) MINITEST_THROW_(stmt, type, MINITEST_FATAL_)

#define MINITEST_NO_THROW_(stmt, MODE)                                                      \
  switch (0) case 0: default: if (::testing::internal::Holder h__{}) {} else                \
    if ([&]() -> bool {                                                                     \
          try { stmt; } catch (const std::exception &e) { h__.text = e.what(); return false; } \
          catch (...) { h__.text = "(not a std::exception)"; return false; }                \
          return true; }()) {} else                                                         \
      MODE(false, std::string("Expected: " #stmt " does not throw\n  Actual: it throws ") + h__.text)
#define EXPECT_NO_THROW(stmt) MINITEST_NO_THROW_(stmt, MINITEST_NONFATAL_)
#define ASSERT_NO_THROW(stmt) MINITEST_NO_THROW_(stmt, MINITEST_FATAL_)

#define FAIL() return ::testing::internal::Voidify() = MINITEST_FAIL_("Failed")
#define SUCCEED() static_cast<void>(0)

#define MINITEST_CLASS_(suite, name) suite##_##name##_Test
#define MINITEST_DEFINE_(suite, name, base)                                                 \
  class MINITEST_CLASS_(suite, name) : public base {                                        \
   public:                                                                                  \
    void TestBody() override;                                                               \
    static void SuiteUp() { base::SetUpTestCase(); }                                        \
    static void SuiteDown() { base::TearDownTestCase(); }                                   \
  };                                                                                        \
  static int minitest_reg_##suite##_##name = ::testing::internal::add_case(                 \
      #suite, #name, []() -> ::testing::Test * { return new MINITEST_CLASS_(suite, name); }, \
      &MINITEST_CLASS_(suite, name)::SuiteUp, &MINITEST_CLASS_(suite, name)::SuiteDown);    \
  void MINITEST_CLASS_(suite, name)::TestBody()

#define TEST_F(fixture, name) MINITEST_DEFINE_(fixture, name, fixture)
#define TEST(suite, name) MINITEST_DEFINE_(suite, name, ::testing::Test)

// Runs every registered case, suite by suite in registration order; argv may carry
// --filter=<substring of Suite.Name>.  Returns the number of failed cases.
int minitest_run_all(int argc, char **argv);
#define RUN_ALL_TESTS() minitest_run_all(0, nullptr)

#ifdef MINITEST_MAIN
namespace testing {
namespace internal {
State &state() {
  static State s;
  return s;
}
}  // namespace internal
}  // namespace testing

int minitest_run_all(int argc, char **argv) {
  using testing::internal::Case;
  using testing::internal::state;
  std::string filter;
  for (int i = 1; i < argc; ++i)
    if (std::strncmp(argv[i], "--filter=", 9) == 0) filter = argv[i] + 9;
  // group by suite, keeping first-appearance order
  std::vector<std::string> suites;
  std::map<std::string, std::vector<const Case *>> by_suite;
  for (const Case &c : state().cases) {
    if (!filter.empty() && (c.suite + "." + c.name).find(filter) == std::string::npos) continue;
    if (!by_suite.count(c.suite)) suites.push_back(c.suite);
    by_suite[c.suite].push_back(&c);
  }
  int ran = 0, failed = 0;
  std::vector<std::string> failed_names;
  for (const std::string &suite : suites) {
    const std::vector<const Case *> &cases = by_suite[suite];
    std::printf("[----------] %zu tests from %s\n", cases.size(), suite.c_str());
    cases.front()->suite_up();
    for (const Case *c : cases) {
      std::printf("[ RUN      ] %s.%s\n", c->suite.c_str(), c->name.c_str());
      std::fflush(stdout);
      state().failures_in_test = 0;
      try {
        testing::Test *t = c->make();
        t->SetUp();
        t->TestBody();
        t->TearDown();
        delete t;
      } catch (const std::exception &e) {
        std::cerr << "unexpected exception: " << e.what() << std::endl;
        ++state().failures_in_test;
      } catch (...) {
        std::cerr << "unexpected exception of unknown type" << std::endl;
        ++state().failures_in_test;
      }
      ++ran;
      if (state().failures_in_test) {
        ++failed;
        failed_names.push_back(c->suite + "." + c->name);
        std::printf("[  FAILED  ] %s.%s\n", c->suite.c_str(), c->name.c_str());
      } else {
        std::printf("[       OK ] %s.%s\n", c->suite.c_str(), c->name.c_str());
      }
    }
    cases.front()->suite_down();
  }
  std::printf("[==========] %d tests ran, %d passed, %d failed\n", ran, ran - failed, failed);
  for (const std::string &n : failed_names) std::printf("[  FAILED  ] %s\n", n.c_str());
  return failed;
}
#endif  // MINITEST_MAIN

#endif  // MINITEST_GTEST_GTEST_H_
