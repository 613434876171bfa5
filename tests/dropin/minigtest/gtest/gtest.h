// A minimal stand-in for <gtest/gtest.h>: just enough of the GoogleTest surface to compile and
// run the reference's own test files (TEST, TEST_F, the EXPECT_/ASSERT_ comparisons they use and
// a main()) on a machine without GoogleTest. Each test executable is a single translation unit,
// so main() lives here. Exit code = number of failed tests (0 = all passed).
#pragma once

#include <cmath>
#include <cstdio>
#include <exception>
#include <functional>
#include <string>
#include <vector>

namespace testing {

class Test {
public:
    virtual ~Test() = default;
    virtual void SetUp() {}
    virtual void TearDown() {}
    virtual void TestBody() = 0;
};

namespace internal {
struct Case {
    std::string name;
    std::function<Test*()> make;
};
inline std::vector<Case>& registry() {
    static std::vector<Case> cases;
    return cases;
}
inline bool& current_failed() {
    static bool failed = false;
    return failed;
}
struct Registrar {
    Registrar(const char* suite, const char* name, std::function<Test*()> make) {
        registry().push_back({std::string(suite) + "." + name, std::move(make)});
    }
};
inline void report(const char* file, int line, const char* what) {
    std::fprintf(stderr, "%s:%d: Failure: %s\n", file, line, what);
    current_failed() = true;
}
}  // namespace internal

inline int RunAllTests() {
    int failed = 0;
    for (auto& c : internal::registry()) {
        internal::current_failed() = false;
        std::printf("[ RUN      ] %s\n", c.name.c_str());
        try {
            Test* t = c.make();
            t->SetUp();
            t->TestBody();
            t->TearDown();
            delete t;
        } catch (const std::exception& e) {
            std::fprintf(stderr, "unexpected exception: %s\n", e.what());
            internal::current_failed() = true;
        } catch (...) {
            std::fprintf(stderr, "unexpected exception\n");
            internal::current_failed() = true;
        }
        std::printf("%s %s\n", internal::current_failed() ? "[  FAILED  ]" : "[       OK ]", c.name.c_str());
        failed += internal::current_failed() ? 1 : 0;
    }
    std::printf("[==========] %zu tests, %d failed\n", internal::registry().size(), failed);
    return failed;
}

}  // namespace testing

#define MINIGTEST_CLASS(suite, name) suite##_##name##_Test
#define MINIGTEST_DEFINE(suite, name, base)                                                              \
    class MINIGTEST_CLASS(suite, name) : public base {                                                   \
    public:                                                                                              \
        void TestBody() override;                                                                        \
    };                                                                                                   \
    static ::testing::internal::Registrar suite##_##name##_registrar(#suite, #name,                      \
        []() -> ::testing::Test* { return new MINIGTEST_CLASS(suite, name)(); });                        \
    void MINIGTEST_CLASS(suite, name)::TestBody()

#define TEST(suite, name) MINIGTEST_DEFINE(suite, name, ::testing::Test)
#define TEST_F(fixture, name) MINIGTEST_DEFINE(fixture, name, fixture)

#define MINIGTEST_CHECK(cond, text, fatal)                                     \
    do {                                                                       \
        if (!(cond)) {                                                         \
            ::testing::internal::report(__FILE__, __LINE__, text);             \
            if (fatal) return;                                                 \
        }                                                                      \
    } while (0)

#define EXPECT_TRUE(c) MINIGTEST_CHECK(static_cast<bool>(c), "EXPECT_TRUE(" #c ")", false)
#define ASSERT_TRUE(c) MINIGTEST_CHECK(static_cast<bool>(c), "ASSERT_TRUE(" #c ")", true)
#define EXPECT_FALSE(c) MINIGTEST_CHECK(!static_cast<bool>(c), "EXPECT_FALSE(" #c ")", false)
#define ASSERT_FALSE(c) MINIGTEST_CHECK(!static_cast<bool>(c), "ASSERT_FALSE(" #c ")", true)
#define EXPECT_EQ(a, b) MINIGTEST_CHECK(static_cast<bool>((a) == (b)), "EXPECT_EQ(" #a ", " #b ")", false)
#define ASSERT_EQ(a, b) MINIGTEST_CHECK(static_cast<bool>((a) == (b)), "ASSERT_EQ(" #a ", " #b ")", true)
#define EXPECT_NE(a, b) MINIGTEST_CHECK(!static_cast<bool>((a) == (b)), "EXPECT_NE(" #a ", " #b ")", false)
#define ASSERT_NE(a, b) MINIGTEST_CHECK(!static_cast<bool>((a) == (b)), "ASSERT_NE(" #a ", " #b ")", true)
#define EXPECT_LT(a, b) MINIGTEST_CHECK((a) < (b), "EXPECT_LT(" #a ", " #b ")", false)
#define EXPECT_GT(a, b) MINIGTEST_CHECK((a) > (b), "EXPECT_GT(" #a ", " #b ")", false)
#define EXPECT_LE(a, b) MINIGTEST_CHECK((a) <= (b), "EXPECT_LE(" #a ", " #b ")", false)
#define EXPECT_GE(a, b) MINIGTEST_CHECK((a) >= (b), "EXPECT_GE(" #a ", " #b ")", false)
#define EXPECT_NEAR(a, b, tol) MINIGTEST_CHECK(std::fabs(static_cast<double>(a) - static_cast<double>(b)) <= (tol), "EXPECT_NEAR(" #a ", " #b ", " #tol ")", false)
#define ASSERT_NEAR(a, b, tol) MINIGTEST_CHECK(std::fabs(static_cast<double>(a) - static_cast<double>(b)) <= (tol), "ASSERT_NEAR(" #a ", " #b ", " #tol ")", true)
#define EXPECT_FLOAT_EQ(a, b) EXPECT_NEAR(a, b, 4e-7 * (std::fabs(static_cast<double>(b)) + 1e-30))
#define EXPECT_THROW(stmt, exc)                                                            \
    do {                                                                                   \
        bool caught__ = false;                                                             \
        try { stmt; } catch (const exc&) { caught__ = true; } catch (...) {}               \
        MINIGTEST_CHECK(caught__, "EXPECT_THROW(" #stmt ", " #exc ")", false);             \
    } while (0)
#define EXPECT_NO_THROW(stmt)                                                              \
    do {                                                                                   \
        bool threw__ = false;                                                              \
        try { stmt; } catch (...) { threw__ = true; }                                      \
        MINIGTEST_CHECK(!threw__, "EXPECT_NO_THROW(" #stmt ")", false);                    \
    } while (0)

#ifndef MINIGTEST_NO_MAIN
int main() { return ::testing::RunAllTests(); }
#endif
