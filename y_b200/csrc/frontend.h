// Minimal front end for the reference's kernel declarations: just enough of
// the `.ysu` grammar to read `[@tile(M, N, K)] kernel name(params) { }` and
// classify the kernel by its parameter list.
#pragma once

#include <string>
#include <vector>

namespace yb {

struct ParamDecl {
    std::string name;
    std::string elem;       // "F16", "F32", ... (element type of GlobalMemory<>, or the scalar type)
    bool is_global = false; // GlobalMemory<elem>
};

struct KernelDecl {
    std::string name;
    bool has_tile = false;
    long long m = 0, n = 0, k = 0;
    std::vector<ParamDecl> params;
};

enum class KernelFamily { None, Invalid, GemmFp8, GemmF16, GemmF16BiasRelu, GemmF16Swiglu, RmsnormResidual, Rope, PagedDecodeAttention };

bool parse_kernels(const std::string& src, std::vector<KernelDecl>* out, std::string* err);
KernelFamily classify_kernel(const KernelDecl& k, std::string* err);
const char* family_name(KernelFamily f);

}  // namespace yb
