"""Golden vectors from the reference's own shader source, compiled as plain C++ on the CPU.

The reference (posedonYT/llama-rs-metal) runs its model through Metal compute shaders
(crates/metal-backend/src/shaders/*.metal). Its host side is Rust for macOS and cannot be
built here, but the shaders are small, scalar and free of graphics state: with a few type
and qualifier definitions (below) they compile with g++ and run one "thread" at a time,
a SIMD group being one lane wide. This script compiles common.metal, the GEMV part of
matrix.metal, elementwise.metal, attention.metal and sampling.metal that way, straight from
a checkout of the reference (nothing of it is copied into this repository), runs the kernels
the Llama path uses on small random inputs, and stores inputs and outputs in
reference_shaders.npz. tests/test_plain.py compares the plain implementation with them.

    python tests/golden/make_golden.py --reference /path/to/llama-rs-metal

Kernels covered (shader file: kernel): elementwise.metal: norm, activation, add, embedding;
matrix.metal: gemv_f32, gemv_bf16; attention.metal: rope, attention, attention_partial,
attention_merge; sampling.metal: argmax.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

SHIM = r"""
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#define kernel
#define device
#define constant const
#define threadgroup static
#define thread
#include <sys/types.h>  // ushort, uint, ulong (64 bits here, as in the shading language)
typedef unsigned char uchar;
static_assert(sizeof(ulong) == 8 && sizeof(uint) == 4 && sizeof(ushort) == 2, "integer widths");
struct uint3 { uint x, y, z; };
struct float4 {
  float v[4];
  float4(float s = 0) { v[0] = v[1] = v[2] = v[3] = s; }
  float& operator[](uint i) { return v[i]; }
};
struct half {  // IEEE binary16, only ever converted to float
  uint16_t bits;
  operator float() const {
    const uint32_t sign = (bits >> 15) & 1u, exponent = (bits >> 10) & 31u, mantissa = bits & 1023u;
    float value;
    if (exponent == 0) value = std::ldexp(static_cast<float>(mantissa), -24);
    else if (exponent == 31) value = mantissa ? NAN : INFINITY;
    else value = std::ldexp(static_cast<float>(mantissa | 1024u), static_cast<int>(exponent) - 25);
    return sign ? -value : value;
  }
};
template <class T, class U> T as_type(U u) {
  static_assert(sizeof(T) == sizeof(U), "as_type needs equal sizes");
  T t;
  std::memcpy(&t, &u, sizeof(T));
  return t;
}
using std::cos; using std::exp; using std::isfinite; using std::max; using std::min; using std::pow; using std::sin;
inline float rsqrt(float x) { return 1.0f / std::sqrt(x); }
// a SIMD group of one lane: every reduction is the identity
inline float simd_sum(float v) { return v; }
inline float4 simd_sum(float4 v) { return v; }
inline float simd_max(float v) { return v; }
inline uint simd_min(uint v) { return v; }
inline bool simd_any(bool v) { return v; }
namespace mem_flags { enum { mem_threadgroup = 0 }; }
inline void threadgroup_barrier(int) {}
"""

HARNESS = r"""
static std::vector<unsigned char> read_file(const std::string& path) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) { std::fprintf(stderr, "cannot read %s\n", path.c_str()); std::exit(2); }
  std::vector<unsigned char> data;
  unsigned char buffer[65536];
  size_t n;
  while ((n = std::fread(buffer, 1, sizeof buffer, f)) > 0) data.insert(data.end(), buffer, buffer + n);
  std::fclose(f);
  return data;
}
static void write_file(const std::string& path, const void* data, size_t bytes) {
  FILE* f = std::fopen(path.c_str(), "wb");
  std::fwrite(data, 1, bytes, f);
  std::fclose(f);
}
// usage: harness DIR CASE ints... ; tensors are DIR/CASE.<name>.bin
int main(int argc, char** argv) {
  const std::string dir = argv[1], name = argv[2];
  std::vector<double> arg;
  for (int i = 3; i < argc; ++i) arg.push_back(std::atof(argv[i]));
  auto in = [&](const char* t) { return read_file(dir + "/" + name + "." + t + ".bin"); };
  auto out = [&](const char* t, const std::vector<float>& v) { write_file(dir + "/" + name + "." + t + ".bin", v.data(), v.size() * 4); };
  P p{};
  if (name == "norm") {            // rows, width, eps, weight type
    const uint rows = arg[0], width = arg[1];
    auto x = in("x"), w = in("w");
    std::vector<float> y(rows * width);
    p.n = width; p.a = width; p.x = arg[2]; p.t = arg[3];
    for (uint r = 0; r < rows; ++r) norm((const float*)x.data(), w.data(), y.data(), p, uint3{r, 0, 0}, 0, 1);
    out("y", y);
  } else if (name == "activation" || name == "add") {
    const uint n = arg[0];
    auto a = in("a"), b = in("b");
    std::vector<float> y(n);
    p.n = n;
    for (uint i = 0; i < n; ++i) {
      if (name == "add") add((const float*)a.data(), (const float*)b.data(), y.data(), p, i);
      else activation((const float*)a.data(), (const float*)b.data(), y.data(), p, i);
    }
    out("y", y);
  } else if (name == "embedding") {  // width, row, weight type
    const uint width = arg[0];
    auto w = in("w");
    std::vector<float> y(width);
    p.n = width; p.a = arg[1]; p.t = arg[2];
    for (uint i = 0; i < width; ++i) embedding(w.data(), y.data(), p, i);
    out("y", y);
  } else if (name == "gemv_f32" || name == "gemv_bf16") {  // tokens, rows, cols
    const uint tokens = arg[0], rows = arg[1], cols = arg[2];
    auto w = in("w"), x = in("x");
    std::vector<float> y(tokens * rows);
    p.a = cols; p.b = rows;
    for (uint t = 0; t < tokens; ++t)
      for (uint gx = 0; gx < (rows + 15) / 16; ++gx)
        for (uint s = 0; s < 4; ++s) {
          if (name == "gemv_f32") gemv_f32(w.data(), (const float*)x.data(), y.data(), p, uint3{gx, t, 0}, s, 0, 1);
          else gemv_bf16(w.data(), (const float*)x.data(), y.data(), p, uint3{gx, t, 0}, s, 0, 1);
        }
    out("y", y);
  } else if (name == "rope") {  // tokens, heads, head_dim, rotary, split_half, start, theta, scale
    const uint tokens = arg[0], heads = arg[1], d = arg[2];
    auto x = in("x"), factors = in("factors");
    std::vector<float> y(tokens * heads * d);
    p.n = tokens * heads * d; p.a = d; p.b = arg[3]; p.c = arg[4]; p.d = arg[5]; p.e = heads; p.x = arg[6]; p.y = arg[7];
    for (uint i = 0; i < p.n; ++i) rope((const float*)x.data(), y.data(), (const float*)factors.data(), p, i);
    out("y", y);
  } else if (name == "attention") {  // tokens, heads, kv_heads, head_dim, start, scale
    const uint tokens = arg[0], heads = arg[1], kv = arg[2], d = arg[3];
    auto q = in("q"), k = in("k"), v = in("v");
    std::vector<float> y(tokens * heads * d);
    p.a = d; p.b = heads; p.c = kv; p.d = arg[4]; p.x = arg[5];
    for (uint t = 0; t < tokens; ++t)
      for (uint h = 0; h < heads; ++h)
        attention((const float*)q.data(), (const float*)k.data(), (const float*)v.data(), y.data(), p, uint3{h, t, 0}, 0, 1);
    out("y", y);
  } else if (name == "attention_decode") {  // heads, kv_heads, head_dim, keys, chunk, scale
    const uint heads = arg[0], kv = arg[1], d = arg[2], keys = arg[3], chunk = arg[4];
    const uint chunks = (keys + chunk - 1) / chunk;
    auto q = in("q"), k = in("k"), v = in("v");
    std::vector<float> partial(heads * chunks * (d + 2)), y(heads * d);
    p.a = d; p.b = heads; p.c = kv; p.d = keys; p.e = chunks; p.f = chunk; p.x = arg[5];
    for (uint h = 0; h < heads; ++h)
      for (uint c = 0; c < chunks; ++c)
        attention_partial((const float*)q.data(), (const float*)k.data(), (const float*)v.data(), partial.data(), p, uint3{h, c, 0}, 0, 1);
    for (uint h = 0; h < heads; ++h) attention_merge(partial.data(), y.data(), p, uint3{h, 0, 0}, 0, 1);
    out("y", y);
  } else if (name == "argmax") {  // n
    auto x = in("x");
    uint result = 0;
    p.n = arg[0];
    argmax((const float*)x.data(), &result, p, 0, 0, 0, 1, uint3{1, 1, 1});
    std::vector<float> y(1, static_cast<float>(static_cast<int>(result)));
    out("y", y);
  } else {
    std::fprintf(stderr, "unknown case %s\n", name.c_str());
    return 2;
  }
  return 0;
}
"""


def bf16_bits(x):
    """float32 array -> uint16 bfloat16 bit patterns (round to nearest even) and the rounded values."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return rounded, (rounded.astype(np.uint32) << 16).view(np.float32)


def build(reference, work):
    shaders = os.path.join(reference, "crates", "metal-backend", "src", "shaders")
    for empty in ("metal_stdlib", "metal_simdgroup_matrix"):   # the shaders' own #include lines
        with open(os.path.join(work, empty), "w") as handle:
            handle.write("namespace metal {}\n")
    with open(os.path.join(shaders, "matrix.metal")) as handle:
        matrix = handle.read()
    gemv_only = matrix[:matrix.index("kernel void expert_mv")]   # the rest needs simdgroup matrices
    with open(os.path.join(work, "matrix_gemv.metal"), "w") as handle:
        handle.write(gemv_only)
    source = os.path.join(work, "harness.cpp")
    with open(source, "w") as handle:
        handle.write(SHIM)
        for name in ("common.metal",):
            handle.write(f'#include "{os.path.join(shaders, name)}"\n')
        handle.write('#include "matrix_gemv.metal"\n')
        for name in ("elementwise.metal", "attention.metal", "sampling.metal"):
            handle.write(f'#include "{os.path.join(shaders, name)}"\n')
        handle.write(HARNESS)
    binary = os.path.join(work, "harness")
    subprocess.run(["g++", "-std=c++17", "-O1", "-w", "-ffp-contract=off", "-I", work, source, "-o", binary], check=True)
    return binary


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--reference", default=os.environ.get("LLAMA_RS_METAL_REFERENCE"),
                        help="checkout of posedonYT/llama-rs-metal")
    parser.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_shaders.npz"))
    args = parser.parse_args()
    if not args.reference:
        sys.exit("give --reference or set LLAMA_RS_METAL_REFERENCE")
    rng = np.random.default_rng(20240607)
    saved = {}
    with tempfile.TemporaryDirectory() as work:
        binary = build(args.reference, work)

        def run(case, tensors, numbers, key=None):
            for name, array in tensors.items():
                np.ascontiguousarray(array).tofile(os.path.join(work, f"{case}.{name}.bin"))
            subprocess.run([binary, work, case] + [repr(float(n)) for n in numbers], check=True)
            y = np.fromfile(os.path.join(work, f"{case}.y.bin"), dtype=np.float32)
            key = key or case
            for name, array in tensors.items():
                saved[f"{key}.{name}"] = array
            saved[f"{key}.args"] = np.asarray(numbers, dtype=np.float64)
            saved[f"{key}.y"] = y
            return y

        f32 = lambda *shape: rng.standard_normal(shape).astype(np.float32)
        # RMSNorm, float32 and bfloat16 weights (weight types 0 and 30 of the shader's val())
        x = f32(5, 24)
        run("norm", {"x": x, "w": (1 + 0.1 * f32(24))}, [5, 24, 1e-5, 0], key="norm_f32")
        bits, _ = bf16_bits(1 + 0.1 * f32(24))
        run("norm", {"x": x, "w": bits}, [5, 24, 1e-6, 30], key="norm_bf16")
        run("activation", {"a": 3 * f32(40), "b": f32(40)}, [40])
        run("add", {"a": f32(17), "b": f32(17)}, [17])
        bits, _ = bf16_bits(f32(6, 12))
        run("embedding", {"w": bits}, [12, 4, 30])
        run("gemv_f32", {"w": f32(21, 40), "x": f32(3, 40)}, [3, 21, 40])
        bits, _ = bf16_bits(f32(35, 24))
        run("gemv_bf16", {"w": bits, "x": f32(2, 24)}, [2, 35, 24])
        # rotation: split-half pairs (the Llama 3 path of the engine), full and partial rotary width,
        # frequency factors as the llama3 rule produces them; and the adjacent-pair form
        factors = np.concatenate([np.ones(3), np.linspace(1.5, 8.0, 5)]).astype(np.float32)
        run("rope", {"x": f32(4 * 3, 16), "factors": factors}, [4, 3, 16, 16, 1, 7, 500000.0, 1.0], key="rope_split")
        run("rope", {"x": f32(2 * 2, 24), "factors": np.ones(6, np.float32)}, [2, 2, 24, 12, 1, 0, 10000.0, 0.25], key="rope_partial")
        run("rope", {"x": f32(3 * 2, 8), "factors": np.ones(4, np.float32)}, [3, 2, 8, 8, 0, 2, 10000.0, 1.0], key="rope_adjacent")
        # prompt attention (grouped queries, with and without earlier keys) and split decode attention
        run("attention", {"q": f32(6, 4, 16), "k": f32(6, 2, 16), "v": f32(6, 2, 16)}, [6, 4, 2, 16, 0, 0.25], key="attention_prompt")
        run("attention", {"q": f32(2, 3, 8), "k": f32(7, 1, 8), "v": f32(7, 1, 8)}, [2, 3, 1, 8, 5, 8 ** -0.5], key="attention_continued")
        run("attention_decode", {"q": f32(4, 16), "k": f32(37, 2, 16), "v": f32(37, 2, 16)}, [4, 2, 16, 37, 8, 0.25])
        # greedy pick: a tie (lowest id wins) and a non-finite logit
        logits = f32(300)
        logits[[41, 250]] = 9.0
        run("argmax", {"x": logits}, [300], key="argmax_tie")
        bad = f32(64)
        bad[10] = np.inf
        run("argmax", {"x": bad}, [64], key="argmax_nonfinite")
    np.savez_compressed(args.out, **saved)
    print(f"wrote {args.out}: {len(saved)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
