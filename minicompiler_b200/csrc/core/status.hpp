#pragma once
// Error-as-value plumbing for the whole host side. Nothing in this library
// throws for control flow: fallible calls hand back a Status or a Result<T>,
// the same convention as the reference (include/minicompiler/result.hpp:14-69).

#include <cassert>
#include <optional>
#include <string>
#include <utility>

namespace minicompiler {

struct Error {
    std::string message;
};

class [[nodiscard]] Status {
public:
    Status() = default;
    Status(Error e) : err_(std::move(e)) {}

    bool ok() const { return !err_.has_value(); }
    const Error& error() const {
        assert(err_.has_value());
        return *err_;
    }
    const std::string& message() const { return error().message; }

private:
    std::optional<Error> err_;
};

template <typename T>
class [[nodiscard]] Result {
public:
    Result(T v) : val_(std::move(v)) {}
    Result(Error e) : err_(std::move(e)) {}

    bool ok() const { return val_.has_value(); }

    T& value() & {
        assert(ok());
        return *val_;
    }
    const T& value() const& {
        assert(ok());
        return *val_;
    }
    T&& value() && {
        assert(ok());
        return std::move(*val_);
    }
    const Error& error() const {
        assert(!ok());
        return *err_;
    }

    T* operator->() { return &value(); }
    const T* operator->() const { return &value(); }
    T& operator*() & { return value(); }
    const T& operator*() const& { return value(); }

    Status status() const { return ok() ? Status() : Status(*err_); }

private:
    std::optional<T> val_;
    std::optional<Error> err_;
};

// Early-return helpers used throughout the host code.
#define MC_TRY(expr)                                   \
    do {                                               \
        ::minicompiler::Status mc_try_st_ = (expr);    \
        if (!mc_try_st_.ok()) return mc_try_st_.error(); \
    } while (0)

#define MC_ASSIGN(lhs, expr)                 \
    auto lhs##_res_ = (expr);                \
    if (!lhs##_res_.ok()) return lhs##_res_.error(); \
    auto lhs = std::move(lhs##_res_).value()

}  // namespace minicompiler
