// tenzo_load_model: weights.bin + model.mlir -> resident engine.
// Replaces TenzoEngineImpl::load_model_from_files (src/runtime/TenzoEngine.cpp:1887-2078 of the reference).
//
// File format, as the reference reads it:
//   weights.bin   fp32 embedding table [vocab][hidden] first; then per layer, in this order,
//                 in_norm f32[h] | q | k | v | attn_sub_norm f32[h] | out | post_norm f32[h] | gate | up |
//                 ffn_sub_norm f32[ffn] | down, and the final norm f32[h] after the last layer. Ternary
//                 matrices are stored as the exporter's [N/4][K] bytes (four rows per byte, 2-bit value+1).
//   model.mlir    optional byte offsets: every  "%c = arith.constant <int> : index" line directly followed by a
//                 "memref.view %buf[%c][] : memref<?xi8> to memref<...>" line names the offset of the next tensor
//                 (the first such pair belongs to the embedding and is skipped); per-matrix scales: every
//                 "%s = arith.constant <float> : f32" line directly followed by a "tenzo.bitlinear_elut"(a, b, %s)
//                 line. Tensors without a view are laid out back to back, matrices without a scale use 1.0.
// Tensors that would run past the end of the file become ones (norms) or zero weights (code 1 everywhere).
//
// Here the file is streamed to the GPU in slabs: the embedding rows are quantised to int8 with per-row
// absmax scales on the device (:1930-1944, same float expressions), and each ternary matrix is repacked from
// the exporter's layout to TL1 by tl1_pack_rows2bit straight into the engine's fused q|k|v and gate|up buffers.
// The reference hard-codes 2560/640 for the projection shapes (:2016-2073); they are taken from the engine
// configuration instead (identical for the BitNet-2B configuration, the only one the reference loads).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <algorithm>
#include <stdexcept>

#include "../../include/tenzo_ext.h"
#include "../../include/tenzo_kernels.h"
#include "common.cuh"
#include "engine.h"

namespace tz {

// ---- manifest text ------------------------------------------------------------------------------
namespace {

std::string trimmed(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r')) ++a;
    while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r')) --b;
    return s.substr(a, b - a);
}

bool word_char(char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_'; }

// "%name = arith.constant <literal> : <type>" -> name (with %), literal. The line may carry text before the
// definition (the reference's patterns are unanchored); the last such definition on the line counts.
bool constant_def(const std::string& line, const char* type, std::string& name, std::string& literal) {
    const std::string key = "arith.constant";
    size_t at = line.rfind(key);
    if (at == std::string::npos) return false;
    size_t eq = line.rfind('=', at);
    if (eq == std::string::npos) return false;
    size_t e = eq;
    while (e > 0 && (line[e - 1] == ' ' || line[e - 1] == '\t')) --e;
    size_t b = e;
    while (b > 0 && word_char(line[b - 1])) --b;
    if (b == 0 || line[b - 1] != '%' || b == e) return false;
    for (size_t i = eq + 1; i < at; ++i)
        if (line[i] != ' ' && line[i] != '\t') return false;
    name = line.substr(b - 1, e - b + 1);
    size_t p = at + key.size();
    if (p >= line.size() || (line[p] != ' ' && line[p] != '\t')) return false;
    while (p < line.size() && (line[p] == ' ' || line[p] == '\t')) ++p;
    size_t q = p;
    while (q < line.size() && line[q] != ' ' && line[q] != '\t' && line[q] != ':') ++q;
    literal = line.substr(p, q - p);
    if (literal.empty()) return false;
    while (q < line.size() && (line[q] == ' ' || line[q] == '\t')) ++q;
    if (q >= line.size() || line[q] != ':') return false;
    ++q;
    while (q < line.size() && (line[q] == ' ' || line[q] == '\t')) ++q;
    const size_t tl = std::strlen(type);
    if (line.compare(q, tl, type) != 0) return false;
    q += tl;
    while (q < line.size() && (line[q] == ' ' || line[q] == '\t' || line[q] == '\r')) ++q;
    return q == line.size();                       // the definition ends the line
}

bool all_digits(const std::string& s) {
    if (s.empty()) return false;
    for (char c : s)
        if (c < '0' || c > '9') return false;
    return true;
}

bool float_literal(const std::string& s) {
    if (s.empty()) return false;
    for (char c : s)
        if (!((c >= '0' && c <= '9') || c == '.' || c == 'e' || c == '+' || c == '-')) return false;
    return true;
}

}  // namespace

void parse_manifest(const std::string& text, std::vector<unsigned long long>& views, std::vector<float>& scales) {
    std::vector<std::string> lines;
    size_t pos = 0;
    while (pos <= text.size()) {
        size_t nl = text.find('\n', pos);
        if (nl == std::string::npos) nl = text.size();
        lines.push_back(text.substr(pos, nl - pos));
        pos = nl + 1;
    }
    for (size_t i = 0; i + 1 < lines.size(); ++i) {
        std::string name, lit;
        const std::string next = trimmed(lines[i + 1]);
        if (constant_def(lines[i], "index", name, lit) && all_digits(lit)) {
            // "%v = memref.view %buf[%name][] : memref<?xi8> to memref<...>"
            const size_t mv = next.find("memref.view");
            if (mv == std::string::npos || next.empty() || next[0] != '%') continue;
            const std::string idx = "[" + name + "][]";
            const size_t at = next.find(idx, mv);
            if (at == std::string::npos) continue;
            const size_t ty = next.find("memref<?xi8>", at);
            if (ty == std::string::npos || next.find("to", ty) == std::string::npos || next.find("memref<", ty + 12) == std::string::npos) continue;
            views.push_back(std::strtoull(lit.c_str(), nullptr, 10));
        } else if (constant_def(lines[i], "f32", name, lit) && float_literal(lit)) {
            // "%y = "tenzo.bitlinear_elut"(a, b, %name)"
            const size_t op = next.find("\"tenzo.bitlinear_elut\"(");
            if (op == std::string::npos || next.empty() || next[0] != '%') continue;
            const size_t close = next.find(')', op);
            if (close == std::string::npos) continue;
            const std::string args = next.substr(op + 23, close - (op + 23));
            const size_t c1 = args.find(','), c2 = c1 == std::string::npos ? c1 : args.find(',', c1 + 1);
            if (c2 == std::string::npos || args.find(',', c2 + 1) != std::string::npos) continue;
            if (trimmed(args.substr(c2 + 1)) != name) continue;
            scales.push_back(std::strtof(lit.c_str(), nullptr));
        }
    }
}

// ---- device side ------------------------------------------------------------------------------------
// One CTA per embedding row: scale = max(|row|, 1e-8)/127, q = clamp(round(x * (1/scale)), +-127)   (:1932-1943)
__global__ void __launch_bounds__(256) embed_quant_rows_kernel(const float* __restrict__ rows, int hidden, int8_t* q, float* scales) {
    __shared__ float s_red[32];
    const float* row = rows + (size_t)blockIdx.x * hidden;
    float amax = 1e-8f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
    amax = block_max(amax, s_red);
    const float scale = amax / 127.0f, inv = 1.0f / scale;
    if (threadIdx.x == 0) scales[blockIdx.x] = scale;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        q[(size_t)blockIdx.x * hidden + i] = (int8_t)(int)fminf(fmaxf(roundf(row[i] * inv), -127.0f), 127.0f);
}

namespace {

struct FileReader {
    FILE* f = nullptr;
    unsigned long long size = 0;
    ~FileReader() { if (f) std::fclose(f); }
    bool open(const char* path) {
        f = std::fopen(path, "rb");
        if (!f) return false;
        if (std::fseek(f, 0, SEEK_END) != 0) return false;
        const long long n = std::ftell(f);
        if (n < 0) return false;
        size = (unsigned long long)n;
        return true;
    }
    bool read_at(unsigned long long off, void* dst, size_t bytes) {
        if (off + bytes > size) return false;
        if (std::fseek(f, (long)off, SEEK_SET) != 0) return false;
        return std::fread(dst, 1, bytes, f) == bytes;
    }
};

}  // namespace

tenzo_status_t load_model_files(Engine& e, const char* weights_path, const char* mlir_path) {
    std::string text;
    {
        FILE* mf = std::fopen(mlir_path, "rb");
        if (!mf) { set_error(std::string("cannot open ") + mlir_path); return TENZO_ERROR_IO; }
        char buf[1 << 16];
        size_t n;
        while ((n = std::fread(buf, 1, sizeof buf, mf)) > 0) text.append(buf, n);
        std::fclose(mf);
    }
    FileReader wf;
    if (!wf.open(weights_path)) { set_error(std::string("cannot open ") + weights_path); return TENZO_ERROR_IO; }

    std::vector<unsigned long long> views;
    std::vector<float> scales;
    parse_manifest(text, views, scales);

    const int h = e.h, qd = e.qd, kvd = e.kvd, ffn = e.ffn, V = e.V;
    const unsigned long long embed_bytes = (unsigned long long)V * h * 4;
    if (wf.size < embed_bytes) { set_error("weights file is shorter than the embedding table"); return TENZO_ERROR_IO; }   // :1898 read failure

    // pinned staging + device staging, sized for the largest matrix / an embedding slab
    const size_t max_raw = (size_t)std::max(std::max(qd, ffn), h) * (size_t)std::max(h, ffn) / 4;
    const int slab_rows = std::max(1, (int)std::min<size_t>((size_t)V, (64u << 20) / ((size_t)h * 4)));
    const size_t stage_bytes = std::max(max_raw, (size_t)slab_rows * h * 4);
    void *h_stage = nullptr, *d_stage = nullptr;
    TZ_CUDA(cudaMallocHost(&h_stage, stage_bytes));
    struct Free { void* h; void* d; ~Free() { cudaFreeHost(h); if (d) cudaFree(d); } } guard{h_stage, nullptr};
    TZ_CUDA(cudaMalloc(&d_stage, stage_bytes));
    guard.d = d_stage;

    // 1. embedding table -> int8 rows + scales (tied LM head)
    if (!e.lm_w) {
        TZ_CUDA(cudaMalloc((void**)&e.lm_w, (size_t)V * h)); e.owned.push_back(e.lm_w);
        TZ_CUDA(cudaMalloc((void**)&e.lm_scales, (size_t)V * 4)); e.owned.push_back(e.lm_scales);
    }
    for (int r0 = 0; r0 < V; r0 += slab_rows) {
        const int rows = std::min(slab_rows, V - r0);
        if (!wf.read_at((unsigned long long)r0 * h * 4, h_stage, (size_t)rows * h * 4)) { set_error("short read in the embedding table"); return TENZO_ERROR_IO; }
        TZ_CUDA(cudaMemcpyAsync(d_stage, h_stage, (size_t)rows * h * 4, cudaMemcpyHostToDevice, e.stream));
        embed_quant_rows_kernel<<<rows, 256, 0, e.stream>>>(static_cast<const float*>(d_stage), h, e.lm_w + (size_t)r0 * h, e.lm_scales + r0);
        TZ_CUDA(cudaGetLastError());
        TZ_CUDA(cudaStreamSynchronize(e.stream));       // the staging buffers are reused
    }

    // 2. layers
    size_t v_idx = 1, s_idx = 0;                         // view 0 is the embedding (:1987)
    unsigned long long seq_off = embed_bytes;
    auto next_offset = [&](unsigned long long bytes) {
        const unsigned long long off = v_idx < views.size() ? views[v_idx++] : seq_off;
        seq_off += bytes;
        return off;
    };
    auto next_scale = [&]() { return s_idx < scales.size() ? scales[s_idx++] : 1.0f; };
    auto load_norm = [&](float*& dst, int n) {
        const unsigned long long off = next_offset((unsigned long long)n * 4);
        float* hbuf = static_cast<float*>(h_stage);
        if (!wf.read_at(off, hbuf, (size_t)n * 4))
            for (int i = 0; i < n; ++i) hbuf[i] = 1.0f;                       // :1967
        if (!dst) { TZ_CUDA(cudaMalloc((void**)&dst, (size_t)n * 4)); e.owned.push_back(dst); }
        TZ_CUDA(cudaMemcpy(dst, hbuf, (size_t)n * 4, cudaMemcpyHostToDevice));
    };
    auto load_ternary = [&](uint8_t* dst, int N, int K) {
        const size_t raw = (size_t)N * K / 4;
        const unsigned long long off = next_offset(raw);
        if (!wf.read_at(off, h_stage, raw)) {
            TZ_CUDA(cudaMemsetAsync(dst, 0x55, raw, e.stream));               // :1983: every weight 0
        } else {
            TZ_CUDA(cudaMemcpyAsync(d_stage, h_stage, raw, cudaMemcpyHostToDevice, e.stream));
            const int rc = tenzo_cuda_tl1_pack_rows2bit(static_cast<const uint8_t*>(d_stage), N, K, dst, e.stream);
            if (rc != 0) throw std::runtime_error("repacking a ternary matrix failed");
        }
        TZ_CUDA(cudaStreamSynchronize(e.stream));
    };
    auto alloc = [&](uint8_t*& p, size_t bytes) {
        if (!p) { TZ_CUDA(cudaMalloc((void**)&p, bytes)); e.owned.push_back(p); }
    };
    const size_t kb = (size_t)h / 4;
    for (int l = 0; l < e.L; ++l) {
        LayerDev& d = e.layers[l];
        alloc(d.qkv, (size_t)(qd + 2 * kvd) * kb);
        alloc(d.o, (size_t)h * qd / 4);
        alloc(d.gateup, (size_t)2 * ffn * kb);
        alloc(d.down, (size_t)h * ffn / 4);
        load_norm(d.in_norm, h);
        load_ternary(d.qkv, qd, h);                      d.s_q = next_scale();
        load_ternary(d.qkv + (size_t)qd * kb, kvd, h);   d.s_k = next_scale();
        load_ternary(d.qkv + (size_t)(qd + kvd) * kb, kvd, h); d.s_v = next_scale();
        load_norm(d.attn_sub_norm, h);
        load_ternary(d.o, h, qd);                        d.s_o = next_scale();
        load_norm(d.post_norm, h);
        load_ternary(d.gateup, ffn, h);                  d.s_gate = next_scale();
        load_ternary(d.gateup + (size_t)ffn * kb, ffn, h); d.s_up = next_scale();
        load_norm(d.ffn_sub_norm, ffn);
        load_ternary(d.down, h, ffn);                    d.s_down = next_scale();
        d.has_mlp = true;
        d.set = true;
    }
    // 3. final norm
    {
        const unsigned long long off = v_idx < views.size() ? views[v_idx] : seq_off;
        float* hbuf = static_cast<float*>(h_stage);
        if (!wf.read_at(off, hbuf, (size_t)h * 4))
            for (int i = 0; i < h; ++i) hbuf[i] = 1.0f;
        if (!e.final_norm) { TZ_CUDA(cudaMalloc((void**)&e.final_norm, (size_t)h * 4)); e.owned.push_back(e.final_norm); }
        TZ_CUDA(cudaMemcpy(e.final_norm, hbuf, (size_t)h * 4, cudaMemcpyHostToDevice));
    }
    e.invalidate_graphs();
    return TENZO_SUCCESS;
}

}  // namespace tz

extern "C" int tenzo_ext_parse_manifest(const char* text, unsigned long long* views, int max_views, int* n_views,
                                        float* scales, int max_scales, int* n_scales) {
    if (!text || !n_views || !n_scales) return TENZO_ERROR_INVALID_ARGUMENT;
    std::vector<unsigned long long> v;
    std::vector<float> s;
    tz::parse_manifest(text, v, s);
    *n_views = (int)v.size();
    *n_scales = (int)s.size();
    for (int i = 0; i < (int)v.size() && i < max_views && views; ++i) views[i] = v[i];
    for (int i = 0; i < (int)s.size() && i < max_scales && scales; ++i) scales[i] = s[i];
    return TENZO_SUCCESS;
}
