// TEST INFRASTRUCTURE ONLY (checker side).  Minimal stand-in for the Jittor
// runtime headers "op.h"/"var.h" so that the reference's own CPU operator
// bodies (jittor_geometric/ops/cpp/*_op.cc, the `#ifdef JIT_cpu` branches) can
// be compiled unmodified, straight from the reference checkout, into
// oracle/_ref/libjgref.so.  Nothing here is reference code: it only supplies
// the few names those bodies touch (Var::ptr<T>(), Var::shape, Op, NanoString,
// NanoVector, DECLARE_jit_run).
#pragma once
#include <cstdint>
#include <cstddef>
#include <cstdlib>
#include <vector>

namespace jittor {

struct NanoString {
    int id;
    constexpr NanoString(int i = 0) : id(i) {}
};
static constexpr NanoString ns_float32{1};
static constexpr NanoString ns_int32{2};

struct NanoVector {
    int64_t v[8];
    int n = 0;
    void push_back(int64_t x) { if (n < 8) v[n++] = x; }
    int64_t operator[](int i) const { return v[i]; }
    int size() const { return n; }
};

struct Var {
    void* mem = nullptr;
    int64_t shape[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int ndim = 0;
    NanoString dt;
    template <class U> U* ptr() { return reinterpret_cast<U*>(mem); }
    NanoString dtype() const { return dt; }
    void set_shape(const NanoVector& s) {
        ndim = s.size();
        for (int i = 0; i < 8; i++) shape[i] = i < s.size() ? s[i] : 0;
    }
};

struct Op {
    virtual ~Op() {}
    virtual const char* name() const = 0;
    virtual void jit_run() = 0;
};

}  // namespace jittor

#define DECLARE_jit_run void jit_run() override
