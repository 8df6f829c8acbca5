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

// Defined by these headers and not by the reference's: code that wants the extensions below the reference's API
// (cached generation, save / load) can test for it and still compile against either set of headers.
#define JASMINE_B200 1

#include <istream>
#include <ostream>

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

// Opt-in: attention layers whose heads are 128 wide run on the tensor cores (bf16 operands, fp32 accumulation, the
// tcgen05 flash kernel) instead of the fp32 kernel that keeps the reference's summation order.  Results then agree with
// the reference to bf16 accuracy (2e-2 of the largest magnitude) instead of 1e-5.  Off by default.
inline bool& attention_bf16() {
    static bool on = false;
    return on;
}

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

// Flat binary record of one tensor: "JSMT", rows, cols (int32), then rows * cols floats in row-major order.
// The reference has no serialisation (mat_t.hpp:322-336 prints text only).
template <typename mat>
void save_tensor(std::ostream& os, const mat& m) {
    const char magic[4] = {'J', 'S', 'M', 'T'};
    const int32_t dims[2] = {(int32_t)m.row_num(), (int32_t)m.col_num()};
    os.write(magic, 4);
    os.write(reinterpret_cast<const char*>(dims), sizeof(dims));
    std::vector<float> v((size_t)dims[0] * dims[1]);
    for (int i = 0; i < dims[0]; ++i)
        for (int j = 0; j < dims[1]; ++j) v[(size_t)i * dims[1] + j] = (float)m(i, j);
    os.write(reinterpret_cast<const char*>(v.data()), (std::streamsize)(v.size() * sizeof(float)));
    if (!os) throw std::runtime_error("save: write failed");
}
// resize: a tensor that the net creates lazily (the gain of a layer norm that never ran) takes the record's shape
template <typename mat>
void load_tensor(std::istream& is, mat& m, bool resize = false) {
    char magic[4];
    int32_t dims[2];
    is.read(magic, 4);
    is.read(reinterpret_cast<char*>(dims), sizeof(dims));
    if (!is || std::memcmp(magic, "JSMT", 4) != 0) throw std::runtime_error("load: not a tensor record");
    if (resize && (dims[0] != m.row_num() || dims[1] != m.col_num())) m = mat(dims[0], dims[1]);
    if (dims[0] != m.row_num() || dims[1] != m.col_num()) throw std::runtime_error("load: tensor shape does not match the net");
    std::vector<float> v((size_t)dims[0] * dims[1]);
    is.read(reinterpret_cast<char*>(v.data()), (std::streamsize)(v.size() * sizeof(float)));
    if (!is) throw std::runtime_error("load: truncated tensor");
    for (int i = 0; i < dims[0]; ++i)
        for (int j = 0; j < dims[1]; ++j) m(i, j) = v[(size_t)i * dims[1] + j];
}

}  // namespace jsm_rt

#endif
