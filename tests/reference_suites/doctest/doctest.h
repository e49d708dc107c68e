// A small stand-in for the doctest framework, enough for the reference's shared
// backend conformance headers (test/backend/backend_conformance_*.hpp) to compile and
// run unmodified against another backend. It implements the assertion macros those
// headers use (CHECK*, REQUIRE*, *_MESSAGE, *_THROWS*, *_NOTHROW, CAPTURE, INFO,
// MESSAGE, FAIL, TEST_CASE), counts failed checks, and aborts a test case at the first
// failed REQUIRE, as the framework does. Not a copy of doctest: no subcases, no
// reporters, no decorators, no stringification of operands beyond operator<<.
#pragma once

#include <cstdio>
#include <exception>
#include <functional>
#include <sstream>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

namespace doctest_shim {

struct RequireFailed final : std::exception {
    const char* what() const noexcept override { return "a REQUIRE failed"; }
};

struct State {
    std::vector<std::pair<const char*, std::function<void()>>> cases;
    unsigned long checks = 0;
    unsigned long failures = 0;
    const char* current = "";
};

inline State& state() {
    static State instance;
    return instance;
}

inline void report(const char* file, int line, const char* kind, const char* text,
                   const std::string& message) {
    State& s = state();
    ++s.failures;
    std::fprintf(stderr, "%s:%d: %s failed in \"%s\": %s%s%s\n", file, line, kind, s.current, text,
                 message.empty() ? "" : " -- ", message.c_str());
}

// Prints a value when it can be streamed, a placeholder otherwise.
template <typename T, typename = void>
struct Streamable : std::false_type {};
template <typename T>
struct Streamable<T, std::void_t<decltype(std::declval<std::ostream&>() << std::declval<const T&>())>>
        : std::true_type {};

template <typename T>
std::string show(const T& value) {
    if constexpr (std::is_enum_v<T>) {
        return std::to_string(static_cast<long long>(value));
    } else if constexpr (Streamable<T>::value) {
        std::ostringstream out;
        out << value;
        return out.str();
    } else {
        return "{?}";
    }
}

struct Registrar {
    Registrar(const char* name, std::function<void()> body) {
        state().cases.emplace_back(name, std::move(body));
    }
};

// Runs every registered case whose name contains `filter` (all when empty). Returns the
// number of failed checks plus escaped exceptions.
inline int run_all(const char* filter) {
    State& s = state();
    unsigned long escaped = 0;
    for (auto& entry : s.cases) {
        if (filter != nullptr && filter[0] != '\0'
                && std::string(entry.first).find(filter) == std::string::npos) {
            continue;
        }
        s.current = entry.first;
        const unsigned long before = s.failures;
        std::fprintf(stderr, "[ case ] %s\n", entry.first);
        try {
            entry.second();
        } catch (const RequireFailed&) {
        } catch (const std::exception& error) {
            ++escaped;
            std::fprintf(stderr, "  exception escaped: %s\n", error.what());
        } catch (...) {
            ++escaped;
            std::fprintf(stderr, "  unknown exception escaped\n");
        }
        std::fprintf(stderr, "[ %s ] %s\n", s.failures == before ? " ok " : "FAIL", entry.first);
    }
    std::fprintf(stderr, "%lu checks, %lu failed, %lu escaped exceptions\n", s.checks, s.failures, escaped);
    return static_cast<int>(s.failures + escaped);
}

}  // namespace doctest_shim

#define DOCTEST_SHIM_CAT2(a, b) a##b
#define DOCTEST_SHIM_CAT(a, b) DOCTEST_SHIM_CAT2(a, b)

#define TEST_CASE(name)                                                                   \
    static void DOCTEST_SHIM_CAT(doctest_shim_case_, __LINE__)();                         \
    static ::doctest_shim::Registrar DOCTEST_SHIM_CAT(doctest_shim_registrar_, __LINE__)( \
            name, &DOCTEST_SHIM_CAT(doctest_shim_case_, __LINE__));                       \
    static void DOCTEST_SHIM_CAT(doctest_shim_case_, __LINE__)()

#define DOCTEST_SHIM_ASSERT(kind, abort_case, condition, text, message_expr)               \
    do {                                                                                   \
        ++::doctest_shim::state().checks;                                                  \
        bool doctest_shim_ok = false;                                                      \
        try {                                                                              \
            doctest_shim_ok = static_cast<bool>(condition);                                \
        } catch (const ::doctest_shim::RequireFailed&) {                                   \
            throw;                                                                         \
        } catch (const std::exception& doctest_shim_error) {                               \
            ::doctest_shim::report(__FILE__, __LINE__, kind, text,                         \
                                   std::string("threw ") + doctest_shim_error.what());     \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
            break;                                                                         \
        }                                                                                  \
        if (!doctest_shim_ok) {                                                            \
            std::ostringstream doctest_shim_message;                                       \
            doctest_shim_message << message_expr;                                          \
            ::doctest_shim::report(__FILE__, __LINE__, kind, text, doctest_shim_message.str()); \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        }                                                                                  \
    } while (false)

#define DOCTEST_SHIM_COMPARE(kind, abort_case, lhs, op, rhs)                               \
    do {                                                                                   \
        ++::doctest_shim::state().checks;                                                  \
        const auto& doctest_shim_lhs = (lhs);                                              \
        const auto& doctest_shim_rhs = (rhs);                                              \
        if (!(doctest_shim_lhs op doctest_shim_rhs)) {                                     \
            ::doctest_shim::report(__FILE__, __LINE__, kind, #lhs " " #op " " #rhs,        \
                                   ::doctest_shim::show(doctest_shim_lhs) + " vs "         \
                                           + ::doctest_shim::show(doctest_shim_rhs));      \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        }                                                                                  \
    } while (false)

#define CHECK(...) DOCTEST_SHIM_ASSERT("CHECK", false, (__VA_ARGS__), #__VA_ARGS__, "")
#define REQUIRE(...) DOCTEST_SHIM_ASSERT("REQUIRE", true, (__VA_ARGS__), #__VA_ARGS__, "")
#define CHECK_FALSE(...) DOCTEST_SHIM_ASSERT("CHECK_FALSE", false, !(__VA_ARGS__), #__VA_ARGS__, "")
#define REQUIRE_FALSE(...) DOCTEST_SHIM_ASSERT("REQUIRE_FALSE", true, !(__VA_ARGS__), #__VA_ARGS__, "")
#define CHECK_MESSAGE(condition, ...) \
    DOCTEST_SHIM_ASSERT("CHECK", false, (condition), #condition, __VA_ARGS__)
#define REQUIRE_MESSAGE(condition, ...) \
    DOCTEST_SHIM_ASSERT("REQUIRE", true, (condition), #condition, __VA_ARGS__)
#define CHECK_FALSE_MESSAGE(condition, ...) \
    DOCTEST_SHIM_ASSERT("CHECK_FALSE", false, !(condition), #condition, __VA_ARGS__)

#define CHECK_EQ(a, b) DOCTEST_SHIM_COMPARE("CHECK_EQ", false, a, ==, b)
#define CHECK_NE(a, b) DOCTEST_SHIM_COMPARE("CHECK_NE", false, a, !=, b)
#define CHECK_LT(a, b) DOCTEST_SHIM_COMPARE("CHECK_LT", false, a, <, b)
#define CHECK_LE(a, b) DOCTEST_SHIM_COMPARE("CHECK_LE", false, a, <=, b)
#define CHECK_GT(a, b) DOCTEST_SHIM_COMPARE("CHECK_GT", false, a, >, b)
#define CHECK_GE(a, b) DOCTEST_SHIM_COMPARE("CHECK_GE", false, a, >=, b)
#define REQUIRE_EQ(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_EQ", true, a, ==, b)
#define REQUIRE_NE(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_NE", true, a, !=, b)
#define REQUIRE_LT(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_LT", true, a, <, b)
#define REQUIRE_LE(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_LE", true, a, <=, b)
#define REQUIRE_GT(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_GT", true, a, >, b)
#define REQUIRE_GE(a, b) DOCTEST_SHIM_COMPARE("REQUIRE_GE", true, a, >=, b)

#define DOCTEST_SHIM_THROWS_ANY(kind, abort_case, expression, text)                       \
    do {                                                                                   \
        ++::doctest_shim::state().checks;                                                  \
        bool doctest_shim_caught = false;                                                  \
        try {                                                                              \
            static_cast<void>(expression);                                                 \
        } catch (...) {                                                                    \
            doctest_shim_caught = true;                                                    \
        }                                                                                  \
        if (!doctest_shim_caught) {                                                        \
            ::doctest_shim::report(__FILE__, __LINE__, kind, text, "");                    \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        }                                                                                  \
    } while (false)

#define DOCTEST_SHIM_THROWS_AS(kind, abort_case, expression, text, ...)                    \
    do {                                                                                   \
        ++::doctest_shim::state().checks;                                                  \
        bool doctest_shim_caught = false;                                                  \
        try {                                                                              \
            static_cast<void>(expression);                                                 \
        } catch (const __VA_ARGS__&) {                                                     \
            doctest_shim_caught = true;                                                    \
        } catch (...) {                                                                    \
        }                                                                                  \
        if (!doctest_shim_caught) {                                                        \
            ::doctest_shim::report(__FILE__, __LINE__, kind, text, "");                    \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        }                                                                                  \
    } while (false)

#define CHECK_THROWS(expression) \
    DOCTEST_SHIM_THROWS_ANY("CHECK_THROWS", false, expression, #expression)
#define REQUIRE_THROWS(expression) \
    DOCTEST_SHIM_THROWS_ANY("REQUIRE_THROWS", true, expression, #expression)
#define CHECK_THROWS_AS(expression, ...) \
    DOCTEST_SHIM_THROWS_AS("CHECK_THROWS_AS", false, expression, #expression " throws " #__VA_ARGS__, \
                           __VA_ARGS__)
#define REQUIRE_THROWS_AS(expression, ...) \
    DOCTEST_SHIM_THROWS_AS("REQUIRE_THROWS_AS", true, expression, #expression " throws " #__VA_ARGS__, \
                           __VA_ARGS__)

#define DOCTEST_SHIM_NOTHROW(kind, abort_case, expression)                                 \
    do {                                                                                   \
        ++::doctest_shim::state().checks;                                                  \
        try {                                                                              \
            static_cast<void>(expression);                                                 \
        } catch (const ::doctest_shim::RequireFailed&) {                                   \
            throw;                                                                         \
        } catch (const std::exception& doctest_shim_error) {                               \
            ::doctest_shim::report(__FILE__, __LINE__, kind, #expression,                  \
                                   std::string("threw ") + doctest_shim_error.what());     \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        } catch (...) {                                                                    \
            ::doctest_shim::report(__FILE__, __LINE__, kind, #expression, "threw");        \
            if (abort_case) throw ::doctest_shim::RequireFailed();                         \
        }                                                                                  \
    } while (false)

#define CHECK_NOTHROW(...) DOCTEST_SHIM_NOTHROW("CHECK_NOTHROW", false, (__VA_ARGS__))
#define REQUIRE_NOTHROW(...) DOCTEST_SHIM_NOTHROW("REQUIRE_NOTHROW", true, (__VA_ARGS__))

#define CAPTURE(...) static_cast<void>(0)
#define INFO(...) static_cast<void>(0)
#define MESSAGE(...)                                              \
    do {                                                          \
        std::ostringstream doctest_shim_message;                  \
        doctest_shim_message << __VA_ARGS__;                      \
        std::fprintf(stderr, "  %s\n", doctest_shim_message.str().c_str()); \
    } while (false)
#define FAIL(...)                                                                         \
    do {                                                                                  \
        std::ostringstream doctest_shim_message;                                          \
        doctest_shim_message << __VA_ARGS__;                                              \
        ::doctest_shim::report(__FILE__, __LINE__, "FAIL", "", doctest_shim_message.str()); \
        throw ::doctest_shim::RequireFailed();                                            \
    } while (false)
#define FAIL_CHECK(...)                                                                   \
    do {                                                                                  \
        std::ostringstream doctest_shim_message;                                          \
        doctest_shim_message << __VA_ARGS__;                                              \
        ::doctest_shim::report(__FILE__, __LINE__, "FAIL_CHECK", "", doctest_shim_message.str()); \
    } while (false)
