"""Generates csrc/interp_gen.h: the PTX interpreter cores of the tiled convolution kernel.

    python tetris-artifact-evalution_b200/csrc/gen_interp.py        (build.py runs this)

The tiled kernel executes a compressed weight PROGRAM (format.h) that is the same for all 32
lanes of a warp.  Each record selects one straight-line block of packed FP32 FMAs
(fma.rn.f32x2) that updates one accumulator row with one column shift of the register-resident
input window; the selection is a jump table (brx.idx.uni), so the accumulators -- K*P2 64-bit
registers -- are only ever named statically.  CUDA C++ cannot express a jump table over code
blocks that share registers (a `switch` is lowered to a compare-and-branch tree, more than ten
branches per record), hence inline PTX, and hence this generator: the blocks differ only in
register names.

For every instantiated (KS, S, K, P2) the header defines Interp<KS,S,K,P2> with
  init()  declares the accumulator registers ta0.. at function scope and zeroes them,
  run()   interprets one program against one staged input tile,
  read()  copies the accumulators into a float2 array for the epilogue.
The register file is shared between the asm statements because PTX registers declared outside
braces live in the enclosing function body; each of the three is emitted once per kernel.

Record dispatch is replicated at the end of every block (threaded code): a block builds the
{w, w} pair, takes the prefetched next record, issues the load of the one after it (programs
are staged in shared memory, so this is a broadcast LDS with a short fixed latency), does its
P2 packed FMAs and jumps straight to the next block.
"""
import os

HERE = os.path.dirname(os.path.abspath(__file__))

# (KS, S, K, P2) instances compiled into the library
CONFIGS = [(3, 1, 16, 4), (3, 2, 16, 4), (1, 1, 16, 4), (1, 2, 16, 4),
           (3, 1, 8, 4), (3, 2, 8, 4), (1, 1, 8, 4), (1, 2, 8, 4)]


def win_cfg(KS, S, P2):
    win = (P2 - 1) * S + KS
    own = P2 * S // 2
    halo = (KS - S + 1) // 2 if KS > S else 0
    assert 2 * (own + halo) >= win and halo <= own
    return win, own, halo


NEXT = ("mov.b32 w, nw; mov.b32 c, nc; ld.shared.v2.u32 {nw, nc}, [pc]; add.u32 pc, pc, 8;")


def gen_run(KS, S, K, P2):
    win, own, halo = win_cfg(KS, S, P2)
    nx = 2 * (own + halo)
    n_fma = K * KS
    labels = ["B%d" % i for i in range(n_fma)] + ["BG", "BE"]
    L = []
    L.append("{")
    L.append(".reg .b32 w, c, nw, nc, icl, rr, t0, a;")
    L.append(".reg .b32 pc;")
    L.append(".reg .b64 w2, xw<%d>;" % nx)
    L.append("mov.b32 pc, %0;")
    L.append("ld.shared.v2.u32 {w, c}, [pc];")
    L.append("ld.shared.v2.u32 {nw, nc}, [pc+8];")
    L.append("add.u32 pc, pc, 16;")
    for i in range(nx):  # defined values even if a malformed program had no GROUP first
        L.append("mov.b64 xw%d, 0;" % i)
    L.append("TS: .branchtargets %s;" % ", ".join(labels))
    L.append("brx.idx.uni c, TS;")
    for k in range(K):
        for s in range(KS):
            L.append("B%d:" % (k * KS + s))
            L.append("mov.b64 w2, {w, w};")
            L.append(NEXT)
            for p in range(P2):
                r = k * P2 + p
                L.append("fma.rn.f32x2 ta%d, w2, xw%d, ta%d;" % (r, p * S + s, r))
            L.append("brx.idx.uni c, TS;")
    # GROUP: payload = (ic_local << 8) | r  ->  load the window of (ic_local, r)
    L.append("BG:")
    L.append("shr.u32 icl, w, 8; and.b32 rr, w, 255;")
    L.append("mul.lo.u32 t0, icl, %3;")
    L.append("mad.lo.u32 a, rr, %4, t0; add.u32 a, a, %1;")
    for j in range(own):
        if j:
            L.append("add.u32 a, a, %6;")
        L.append("ld.shared.v2.b64 {xw%d, xw%d}, [a];" % (2 * j, 2 * j + 1))
    if halo:
        L.append("mad.lo.u32 a, rr, %5, t0; add.u32 a, a, %2;")
        for j in range(halo):
            if j:
                L.append("add.u32 a, a, %7;")
            L.append("ld.shared.v2.b64 {xw%d, xw%d}, [a];" % (2 * (own + j), 2 * (own + j) + 1))
    L.append(NEXT)
    L.append("brx.idx.uni c, TS;")
    L.append("BE:")
    L.append("}")
    return L


def c_string(lines):
    return "\n".join('      "%s\\n"' % ln for ln in lines)


def gen_struct(KS, S, K, P2):
    nacc = K * P2
    out = []
    out.append("template <> struct Interp<%d, %d, %d, %d> {" % (KS, S, K, P2))
    init = [".reg .b64 ta<%d>;" % nacc] + ["mov.b64 ta%d, 0;" % i for i in range(nacc)]
    out.append("  static __device__ __forceinline__ void init() {")
    out.append("    asm volatile(\n%s);" % c_string(init))
    out.append("  }")
    out.append("  // %0 program (shared-space address), %1 own window base, %2 halo window base, %3 channel pitch, %4 row pitch,")
    out.append("  // %5 halo row pitch, %6 chunk-plane pitch, %7 halo chunk pitch (all shared-space bytes)")
    out.append("  static __device__ __forceinline__ void run(uint32_t prog, uint32_t a_own0, uint32_t a_halo0,")
    out.append("      uint32_t icpitch, uint32_t rp, uint32_t halo_rp, uint32_t cp16, uint32_t halo_js) {")
    out.append("    asm volatile(\n%s" % c_string(gen_run(KS, S, K, P2)))
    out.append('      :: "r"(prog), "r"(a_own0), "r"(a_halo0), "r"(icpitch), "r"(rp), "r"(halo_rp),')
    out.append('         "r"(cp16), "r"(halo_js) : "memory");')
    out.append("  }")
    out.append("  static __device__ __forceinline__ void read(float2 (&acc)[%d][%d]) {" % (K, P2))
    for k in range(K):
        for p in range(P2):
            out.append('    asm volatile("mov.b64 {%%0, %%1}, ta%d;" : "=f"(acc[%d][%d].x), "=f"(acc[%d][%d].y));'
                       % (k * P2 + p, k, p, k, p))
    out.append("  }")
    out.append("};")
    return "\n".join(out)


def generate():
    parts = ["// GENERATED by gen_interp.py -- do not edit; edit the generator.",
             "#pragma once", "#include <stdint.h>", "", "namespace tetris {", "",
             "template <int KS, int S, int K, int P2> struct Interp;", ""]
    for cfg in CONFIGS:
        parts.append(gen_struct(*cfg))
        parts.append("")
    parts.append("}  // namespace tetris")
    return "\n".join(parts) + "\n"


def write(path=None):
    path = path or os.path.join(HERE, "interp_gen.h")
    text = generate()
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as fh:
            fh.write(text)
    return path


if __name__ == "__main__":
    print(write())
