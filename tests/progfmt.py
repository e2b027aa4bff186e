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


LIST_HEADER_WORDS = 4
LIST_TAIL_UNITS = 2


def pack_lists(w, K=16, TIC=16):
    """Dense OIHW float32 -> (units uint64[], piece_offsets int32[B*T+1]) of the LIST form:
    per piece K counts + total + 3 zero words, then the K lists of {weight, pos} records in
    (ic, r, s) order, each padded to an even length with {0, TIC << 8}, then two such records as
    sentinels; pieces padded to an even number of 8-byte units."""
    w = np.ascontiguousarray(w, np.float32)
    OC, IC, KS, _ = w.shape
    B, T = -(-OC // K), -(-IC // TIC)
    bits = w.view(np.uint32)
    words, offsets = [], [0]           # 32-bit words; two per unit
    for b in range(B):
        for t in range(T):
            start = len(words)
            counts, recs = [], []
            for k in range(K):
                oc = b * K + k
                n = 0
                if oc < OC:
                    blk = w[oc, t * TIC:(t + 1) * TIC]           # [icl][r][s]
                    for icl, r, s in zip(*np.nonzero(blk != 0)):  # row-major = (ic, r, s) order
                        recs += [int(bits[oc, t * TIC + icl, r, s]), (int(icl) << 8) | (int(r) << 4) | int(s)]
                        n += 1
                if n % 2:                       # lists are padded to an even length
                    recs += [0, TIC << 8]
                    n += 1
                counts.append(n)
            words += counts + [sum(counts), 0, 0, 0] + recs + [0, TIC << 8] * 2
            while ((len(words) - start) // 2) % PROG_ALIGN_OPS:
                words += [0, TIC << 8]
            offsets.append(len(words) // 2)
    words += [0, TIC << 8] * LIST_TAIL_UNITS
    return np.array(words, np.uint32).view(np.uint64), np.array(offsets, np.int32)


def unpack_lists(units, offsets, OC, IC, KS, K=16, TIC=16):
    """LIST form -> dense OIHW float32."""
    B, T = -(-OC // K), -(-IC // TIC)
    words = np.ascontiguousarray(units).view(np.uint32)
    w = np.zeros((OC, IC, KS, KS), np.uint32)
    for b in range(B):
        for t in range(T):
            base = 2 * int(offsets[b * T + t])
            counts = words[base:base + K]
            assert int(words[base + K]) == int(counts.sum())
            i = base + K + LIST_HEADER_WORDS
            for k in range(K):
                for _ in range(int(counts[k])):
                    val, pos = int(words[i]), int(words[i + 1])
                    i += 2
                    if pos == TIC << 8:
                        assert val == 0  # a padding record
                        continue
                    w[b * K + k, t * TIC + (pos >> 8), (pos >> 4) & 15, pos & 15] = val
            assert words[i] == 0 and words[i + 1] == TIC << 8  # the sentinels
    return w.view(np.float32)


# ---- compressed-filter files (tetris_filter_save / _load / _file_check) ----------------------
FILE_MAGIC = b"TETRISF1"
FILE_VERSION = 1
FILE_HEADER = "<8sII" + "i" * 12 + "qqq" + "QQ"   # see FileHeader in csrc/serialize.cu
TUNED_INTS = 9


def fnv1a(data):
    h = 1469598103934665603
    for byte in data:
        h = ((h ^ byte) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def write_filter_file(path, w, K=8, TIC=16, tuned=(), damage=None):
    """Checker-side writer of the file format: what tetris_filter_save must produce for the dense
    OIHW filter `w` (groups == 1).  `damage(header_fields, payload) -> (header_fields, payload)`
    lets a test corrupt the file before it is written."""
    import struct
    w = np.ascontiguousarray(w, np.float32)
    OC, IC, KS, _ = w.shape
    B, T = -(-OC // K), -(-IC // TIC)
    ops, poffs, nnz = pack(w, K, TIC)
    units, loffs = pack_lists(w, K, TIC)
    tuned = np.asarray(tuned, np.int32).reshape(-1, TUNED_INTS)
    payload = loffs.tobytes() + poffs.tobytes() + units.tobytes() + ops.tobytes() + tuned.tobytes()
    fields = dict(in_channel=IC, out_channel=OC, kernel_size=KS, groups=1, oc_block=K, tile_ic=TIC,
                  n_oc_blocks=B, n_stages=T, max_prog_ops=int(np.diff(poffs).max()),
                  max_list_units=int(np.diff(loffs).max()), deterministic=0, n_tuned=len(tuned),
                  nnz=nnz, n_ops=ops.size, n_list_units=units.size)
    if damage:
        fields, payload = damage(fields, payload)
    fields.setdefault("payload_bytes", len(payload))
    fields.setdefault("checksum", fnv1a(payload))
    header = struct.pack(FILE_HEADER, fields.get("magic", FILE_MAGIC), fields.get("version", FILE_VERSION),
                         struct.calcsize(FILE_HEADER),
                         *[fields[k] for k in ("in_channel", "out_channel", "kernel_size", "groups", "oc_block",
                                               "tile_ic", "n_oc_blocks", "n_stages", "max_prog_ops",
                                               "max_list_units", "deterministic", "n_tuned", "nnz", "n_ops",
                                               "n_list_units", "payload_bytes", "checksum")])
    with open(path, "wb") as fh:
        fh.write(header + payload)
    return header, payload
