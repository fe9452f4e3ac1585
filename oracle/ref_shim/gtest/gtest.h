// Minimal stand-in for <gtest/gtest.h>, only so that the reference's
// tests/test_util.cpp (its double-precision evaluator and random-graph
// generator) compiles unmodified where GoogleTest is not installed.
// TEST INFRASTRUCTURE ONLY: nothing in the product includes this.
#pragma once
#include <iostream>
#include <sstream>
#include <string>

namespace testing {

class AssertionResult {
public:
    explicit AssertionResult(bool ok) : ok_(ok) {}
    AssertionResult(const AssertionResult& o) : ok_(o.ok_), text_(o.text_.str()) {}
    explicit operator bool() const { return ok_; }
    std::string message() const { return text_.str(); }
    template <typename T>
    AssertionResult& operator<<(const T& v) {
        text_ << v;
        return *this;
    }

private:
    bool ok_;
    std::ostringstream text_;
};

inline AssertionResult AssertionSuccess() { return AssertionResult(true); }
inline AssertionResult AssertionFailure() { return AssertionResult(false); }

struct FailureSink {
    ~FailureSink() { std::cerr << "ref_shim: reference test utility reported a failure: " << text.str() << std::endl; }
    template <typename T>
    FailureSink& operator<<(const T& v) {
        text << v;
        return *this;
    }
    std::ostringstream text;
};

}  // namespace testing

#define ADD_FAILURE() ::testing::FailureSink()
