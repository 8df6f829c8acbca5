// Glue between the jasmine-style headers and the C ABI of libjasmine_b200.so:
// status -> exception mapping, the expression-program builder, small RAII helpers.
#ifndef JASMINE_B200_RUNTIME_HPP_
#define JASMINE_B200_RUNTIME_HPP_

#include <cstdint>
#include <cstring>
#include <memory>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "jasmine_b200.h"

namespace jsm_rt {

// The reference reports errors with exceptions only: std::invalid_argument for a dot-product shape
// mismatch (mat_express_t.hpp:709-712), std::runtime_error for everything else (mat_mha_t.hpp:268-269).
inline void check(jsm_status s) {
    if (s == JSM_OK) return;
    std::string msg = jsm_last_error();
    if (s == JSM_INVALID_ARG) throw std::invalid_argument(msg);
    if (s == JSM_OOM) throw std::bad_alloc();
    throw std::runtime_error(msg);
}

inline void* stream() { return nullptr; }

struct device_buffer {
    void* p = nullptr;
    explicit device_buffer(size_t bytes) { check(jsm_malloc(&p, bytes)); }
    device_buffer(const device_buffer&) = delete;
    device_buffer& operator=(const device_buffer&) = delete;
    ~device_buffer() { jsm_free(p); }
};

// Postfix program under construction.  Identical operands are stored once, so an expression may
// mention the same matrix many times and still fit the leaf table.
struct builder {
    std::vector<jsm_instr> prog;
    std::vector<jsm_mat> leaves;
    std::vector<std::shared_ptr<void>> keep;  // temporaries that must outlive the launch

    void leaf(const jsm_mat& m) {
        int idx = -1;
        for (size_t i = 0; i < leaves.size(); ++i) {
            const jsm_mat& o = leaves[i];
            if (o.data == m.data && o.rows == m.rows && o.cols == m.cols && o.row_stride == m.row_stride &&
                o.col_stride == m.col_stride && o.dtype == m.dtype) {
                idx = (int)i;
                break;
            }
        }
        if (idx < 0) {
            if (leaves.size() >= JSM_MAX_LEAVES) throw std::runtime_error("expression has more than 8 distinct operands: materialise a part with clone()");
            leaves.push_back(m);
            idx = (int)leaves.size() - 1;
        }
        prog.push_back(jsm_instr{JSM_OP_LEAF, idx, 0.0f});
    }
    void imm(float v) { prog.push_back(jsm_instr{JSM_OP_IMM, 0, v}); }
    void op(int code, float v = 0.0f) {
        if (prog.size() >= JSM_MAX_INSTR) throw std::runtime_error("expression is longer than 32 operations: materialise a part with clone()");
        prog.push_back(jsm_instr{code, 0, v});
    }
};

}  // namespace jsm_rt

#endif
