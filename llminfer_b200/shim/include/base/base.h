// Host-side mirror of the reference engine's base vocabulary, limited to what its attention
// operator boundary uses: device / data type enums, Status, NoCopyable and the abort-on-failure
// check the reference gets from glog. Same names and values as code/include/base/base.h:44-58,
// :90-124 of the reference project, so call sites written against it compile unchanged.
#ifndef LLMINFER_SHIM_BASE_BASE_H
#define LLMINFER_SHIM_BASE_BASE_H

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>

// The reference aborts through glog's CHECK; without glog the same contract is kept with a
// message on stderr and std::abort().
#ifndef CHECK
#define LLMINFER_SHIM_OWN_CHECK 1
#define CHECK(cond)                                                                          \
    do {                                                                                     \
        if (!(cond)) {                                                                       \
            std::fprintf(stderr, "%s:%d] Check failed: %s\n", __FILE__, __LINE__, #cond);    \
            std::abort();                                                                    \
        }                                                                                    \
    } while (0)
#endif

#ifndef UNUSED
#define UNUSED(expr) do { (void)(expr); } while (0)
#endif

namespace base {

enum class DeviceType : uint8_t { DeviceUnknown = 0, DeviceCUDA = 1, DeviceCPU = 2 };

enum class DataType : uint8_t {
    DataTypeUnknown = 0,
    DataTypeFp32 = 1,
    DataTypeBf16 = 2,
    DataTypeFp16 = 3,
    DataTypeInt32 = 4,
    DataTypeInt4x8 = 5,
};

inline size_t data_type_size(DataType t) {
    switch (t) {
        case DataType::DataTypeBf16:
        case DataType::DataTypeFp16: return 2;
        case DataType::DataTypeFp32:
        case DataType::DataTypeInt32:
        case DataType::DataTypeInt4x8: return 4;
        default: CHECK(false && "unknown data type"); return 0;
    }
}

class NoCopyable {
protected:
    NoCopyable() = default;
    ~NoCopyable() = default;
    NoCopyable(const NoCopyable&) = delete;
    NoCopyable& operator=(const NoCopyable&) = delete;
};

enum class StatusCode : uint8_t {
    Success = 0,
    FunctionUnImplement = 1,
    PathNotValid = 2,
    ModelParseError = 3,
    InternalError = 5,
    KeyValueHasExist = 6,
    InvalidArgument = 7,
};

class Status {
public:
    Status(StatusCode code = StatusCode::Success, std::string msg = "")
        : code_(code), msg_(std::move(msg)) {}
    bool operator==(StatusCode code) const { return code_ == code; }
    bool operator!=(StatusCode code) const { return code_ != code; }
    operator int() const { return static_cast<int>(code_); }
    operator bool() const { return code_ == StatusCode::Success; }
    StatusCode get_err_code() const { return code_; }
    const std::string& get_err_msg() const { return msg_; }
    void set_err_msg(const std::string& msg) { msg_ = msg; }

private:
    StatusCode code_;
    std::string msg_;
};

namespace error {
inline Status success(const std::string& msg = "") { return Status(StatusCode::Success, msg); }
inline Status invalid_argument(const std::string& msg = "") {
    return Status(StatusCode::InvalidArgument, msg);
}
inline Status internal_error(const std::string& msg = "") {
    return Status(StatusCode::InternalError, msg);
}
inline Status function_not_implement(const std::string& msg = "") {
    return Status(StatusCode::FunctionUnImplement, msg);
}
}  // namespace error

}  // namespace base

// Model code wraps layer calls like this (code/include/base/base.h:127-137).
#define STATUS_CHECK(call)                                                                   \
    do {                                                                                     \
        const base::Status& status_ = (call);                                                \
        if (!status_) {                                                                      \
            std::fprintf(stderr, "Infer error\n File: %s Line: %d\n Error code: %d\n Error " \
                         "msg: %s\n", __FILE__, __LINE__, int(status_),                      \
                         status_.get_err_msg().c_str());                                     \
            std::abort();                                                                    \
        }                                                                                    \
    } while (0)

#endif  // LLMINFER_SHIM_BASE_BASE_H
