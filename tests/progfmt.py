"""Checker-side restatement (numpy) of the compressed program format.

`pack()` builds, on the CPU, the record stream that the device compressor must emit for a dense
filter -- bit for bit (it is integer and bit-pattern work).  `unpack()` turns a stream back into
a dense filter (the compress -> decompress round trip).  Used by tests only.
"""
import numpy as np

PROG_ALIGN_OPS = 2
TAIL_PAD_OPS = 16


def pack(w, K=16, TIC=16):
    """Dense OIHW float32 -> (ops uint64[], prog_offsets int32[B*T+1], nnz)."""
    w = np.ascontiguousarray(w, np.float32)
    OC, IC, KS, _ = w.shape
    B, T = -(-OC // K), -(-IC // TIC)
    c_group, c_end = K * KS, K * KS + 1
    bits = w.view(np.uint32)
    ops, offsets, nnz = [], [0], 0
    for b in range(B):
        for t in range(T):
            n0 = len(ops)
            for icl in range(TIC):
                ic = t * TIC + icl
                if ic >= IC:
                    break
                for r in range(KS):
                    blk = w[b * K:(b + 1) * K, ic, r, :]        # [k][s]
                    ks, ss = np.nonzero(blk != 0)
                    if ks.size == 0:
                        continue
                    ops.append((c_group << 32) | (icl << 8) | r)
                    for k, s in zip(ks.tolist(), ss.tolist()):   # row-major = (k, s) order
                        ops.append(((k * KS + s) << 32) | int(bits[b * K + k, ic, r, s]))
                    nnz += ks.size
            ops.append(c_end << 32)
            while (len(ops) - n0) % PROG_ALIGN_OPS:
                ops.append(c_end << 32)
            offsets.append(len(ops))
    ops.extend([c_end << 32] * TAIL_PAD_OPS)
    return np.array(ops, np.uint64), np.array(offsets, np.int32), nnz


def unpack(ops, offsets, OC, IC, KS, K=16, TIC=16):
    """Record stream -> dense OIHW float32 (inverse of pack / of the device compressor)."""
    B, T = -(-OC // K), -(-IC // TIC)
    c_group, c_end = K * KS, K * KS + 1
    w = np.zeros((OC, IC, KS, KS), np.uint32)
    for b in range(B):
        for t in range(T):
            i = int(offsets[b * T + t])
            ic = r = None
            while True:
                op = int(ops[i]); i += 1
                code, payload = op >> 32, op & 0xFFFFFFFF
                if code == c_end:
                    break
                if code == c_group:
                    ic, r = t * TIC + (payload >> 8), payload & 255
                    continue
                k, s = divmod(code, KS)
                w[b * K + k, ic, r, s] = payload
    return w.view(np.float32)
