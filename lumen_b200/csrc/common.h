// Shared host-side helpers: thread-local error message, dtype table, status-returning guards.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/lumen_b200.h"

namespace lb {

struct Error : std::runtime_error {
    int status;
    Error(int status, const std::string& what) : std::runtime_error(what), status(status) {}
};

void set_last_error(const std::string& message);

std::string format(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

[[noreturn]] inline void fail(int status, const std::string& message) { throw Error(status, message); }

// Runs `f`, mapping exceptions to a status code and the thread's last-error message.
template <class F>
int guarded(F f) {
    try {
        f();
        return LB_OK;
    } catch (const Error& e) {
        set_last_error(e.what());
        return e.status;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return LB_ERR_INVALID;
    }
}

const char* dtype_name(int dtype);
int dtype_from_name(const std::string& name);  // throws on unknown
int dtype_size(int dtype);
inline bool dtype_is_float(int d) { return d >= LB_F16; }
inline bool dtype_is_signed(int d) { return d >= LB_I8 && d <= LB_I64; }
inline bool dtype_is_unsigned(int d) { return d >= LB_U8 && d <= LB_U64; }

int64_t numel(const std::vector<int64_t>& shape);
// Throws unless `t` is dense row-major of `dtype` and `shape`.
void check_dense(const lb_tensor& t, int dtype, const std::vector<int64_t>& shape, const char* what);

}  // namespace lb
