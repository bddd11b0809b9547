"""Numpy model of the B200 stream layout and of how one warp consumes it.

Test infrastructure: an independent restatement (from the layout description in
csrc/cq_common.cuh) of
  * the re-pack reference buffers -> stream (`build_blob`), and
  * the decode + mma.sync.m16n8k16 fragment walk of the matvec kernel
    (`consume_blob`), including the fp16 exponent-trick decode with the same masks
    and constants as the CUDA code.
CPU tests check model(build) against the oracle; GPU tests check the CUDA re-pack
against `build_blob` byte for byte.
"""
import numpy as np

PAD = 0xFFFF


def dims(bits, K, N, C, G):
    if G == -1:
        G = K
    Kc = K - C
    n_gran = (Kc + 127) // 128
    d = dict(bits=bits, K=K, N=N, C=C, G=G, Kc=Kc, n_gran=n_gran, Kp=n_gran * 128,
             Cp=(C + 15) // 16 * 16, n_sub=(N + 15) // 16, sets=2 if G == 64 else 1)
    d["gran_bytes"] = 256 * bits + d["sets"] * 32
    d["cher_bytes"] = d["Cp"] // 16 * 512

    def al(x):
        return (x + 255) & ~255
    off = 0
    d["off_stream"] = off
    off = al(off + d["n_sub"] * n_gran * d["gran_bytes"])
    d["off_cherry"] = off
    off = al(off + d["n_sub"] * d["cher_bytes"])
    d["off_perm"] = off
    off = al(off + d["Kp"] * 2)
    d["off_cidx"] = off
    off = al(off + (d["Cp"] or 16) * 2)
    d["blob_bytes"] = off
    return d


def ref_codes(qweight, bits):
    """(K', N) unsigned codes from the reference's uint8 rows."""
    q = qweight.astype(np.uint32)
    r, n = q.shape
    if bits == 4:
        out = np.empty((2 * r, n), np.uint32)
        out[0::2] = q & 15
        out[1::2] = q >> 4
        return out
    t = q.reshape(r // 3, 3, n)
    w = t[:, 0] | (t[:, 1] << 8) | (t[:, 2] << 16)
    return np.stack([(w >> (3 * i)) & 7 for i in range(8)], axis=1).reshape(r // 3 * 8, n)


def s4_shift(i):
    return 4 * ((i >> 1) + 4 * (i & 1))


def build_blob(qweight, scales, cherry_weight, cherry_indices, bits, K, G):
    N = qweight.shape[1]
    C = len(cherry_indices)
    d = dims(bits, K, N, C, G)
    G = d["G"]
    u = np.zeros((d["Kp"], d["n_sub"] * 16), np.uint32)
    u[:d["Kc"], :N] = ref_codes(qweight, bits)
    blob = np.zeros(d["blob_bytes"], np.uint8)
    gb = d["gran_bytes"]
    sc16 = scales.view(np.uint16)
    for sub in range(d["n_sub"]):
        for gi in range(d["n_gran"]):
            base = d["off_stream"] + (sub * d["n_gran"] + gi) * gb
            words = np.zeros(64 * bits, np.uint32)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for hi in range(2):
                    n = sub * 16 + g + 8 * hi
                    if bits == 4:
                        for h in range(2):
                            for half in range(2):
                                w = 0
                                for i in range(8):
                                    kc = gi * 128 + 64 * h + 16 * t + 8 * half + i
                                    w |= int(u[kc, n]) << s4_shift(i)
                                words[(h * 128 + lane * 4) + 2 * hi + half] = w
                    else:
                        ws = [0, 0, 0]
                        for e in range(32):
                            kc = gi * 128 + 16 * t + (e if e < 16 else 64 + e - 16)
                            code = int(u[kc, n])
                            if e < 30:
                                q = e >> 1
                                ws[q // 5] |= code << (16 * (e & 1) + 1 + 3 * (q % 5))
                            else:
                                for wi in range(3):
                                    ws[wi] |= ((code >> wi) & 1) << (16 * (e & 1))
                        for wi in range(3):
                            words[lane * 6 + 3 * hi + wi] = ws[wi]
            blob[base:base + 256 * bits] = words.view(np.uint8)
            srow = np.zeros(d["sets"] * 16, np.uint16)
            for sp in range(d["sets"]):
                kc0 = gi * 128 + sp * (128 // d["sets"])
                for r in range(16):
                    n = sub * 16 + r
                    if n < N and kc0 < d["Kc"]:
                        srow[sp * 16 + r] = sc16[kc0 // G, n]
            blob[base + 256 * bits: base + gb] = srow.view(np.uint8)
    cw16 = cherry_weight.view(np.uint16) if C else np.zeros((0, N), np.uint16)
    for sub in range(d["n_sub"]):
        for j in range(d["Cp"] // 16):
            blk = np.zeros((32, 8), np.uint16)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for reg in range(4):
                    for e in range(2):
                        c = 16 * j + 2 * t + e + 8 * (reg >> 1)
                        n = sub * 16 + g + 8 * (reg & 1)
                        if c < C and n < N:
                            blk[lane, 2 * reg + e] = cw16[c, n]
            o = d["off_cherry"] + sub * d["cher_bytes"] + j * 512
            blob[o:o + 512] = blk.reshape(-1).view(np.uint8)
    perm = np.full(d["Kp"], PAD, np.uint16)
    idx = cherry_indices.astype(np.int64)
    mask = np.ones(K, bool)
    mask[idx] = False
    perm[:d["Kc"]] = np.nonzero(mask)[0]
    blob[d["off_perm"]:d["off_perm"] + 2 * d["Kp"]] = perm.view(np.uint8)
    cidx = np.full(d["Cp"] or 16, PAD, np.uint16)
    cidx[:C] = idx
    if d["Cp"] == 0:
        cidx[:] = 0   # never written by the re-pack; compare only Cp entries
    blob[d["off_cidx"]:d["off_cidx"] + 2 * d["Cp"]] = cidx[:d["Cp"]].view(np.uint8)
    return blob, d


# ------------------------------------------------------------------ consumption model
MAGIC = 0x64006400


def _hfma2(a_u32, mul, add):
    """fma.rn.f16x2 on a packed pair: result as two float32 (exact for these inputs)."""
    pair = np.array([a_u32 & 0xFFFF, a_u32 >> 16], np.uint16).view(np.float16).astype(np.float64)
    r = pair * mul + add
    return r.astype(np.float16).astype(np.float64)


def dequant4(w):
    v1, v2 = (w << 2) & 0xFFFFFFFF, w >> 6
    return [
        _hfma2((v1 & 0x003C003C) | MAGIC, 0.25, -263.5),
        _hfma2((v1 & 0x03C003C0) | MAGIC, 1 / 64, -23.5),
        _hfma2((v2 & 0x003C003C) | MAGIC, 0.25, -263.5),
        _hfma2((v2 & 0x03C003C0) | MAGIC, 1 / 64, -23.5),
    ]


def dequant3(w0, w1, w2):
    out = []
    for w in (w0, w1, w2):
        v = w >> 9
        out.append(_hfma2((w & 0x000E000E) | MAGIC, 0.5, -515.5))
        out.append(_hfma2((w & 0x00700070) | MAGIC, 1 / 16, -67.5))
        out.append(_hfma2((w & 0x03800380) | MAGIC, 1 / 128, -11.5))
        out.append(_hfma2((v & 0x000E000E) | MAGIC, 0.5, -515.5))
        out.append(_hfma2((v & 0x00700070) | MAGIC, 1 / 16, -67.5))
    r = (((w0 << 1) & 0x00020002) | MAGIC) | ((w1 << 2) & 0x00040004) | ((w2 << 3) & 0x00080008)
    out.append(_hfma2(r, 0.5, -515.5))
    return out


def consume_blob(blob, d, x):
    """y (M, N) float64 computed the way the kernel walks the stream."""
    bits, N, M = d["bits"], d["N"], x.shape[0]
    perm = blob[d["off_perm"]:d["off_perm"] + 2 * d["Kp"]].view(np.uint16)
    cidx = blob[d["off_cidx"]:d["off_cidx"] + 2 * d["Cp"]].view(np.uint16)
    xs = np.zeros((M, d["Kp"]))
    ok = perm != PAD
    xs[:, ok] = x[:, perm[ok].astype(np.int64)].astype(np.float64)
    xc = np.zeros((M, d["Cp"]))
    okc = cidx != PAD
    xc[:, okc] = x[:, cidx[okc].astype(np.int64)].astype(np.float64)
    y = np.zeros((M, d["n_sub"] * 16))
    gb = d["gran_bytes"]
    for sub in range(d["n_sub"]):
        for gi in range(d["n_gran"]):
            base = d["off_stream"] + (sub * d["n_gran"] + gi) * gb
            words = blob[base:base + 256 * bits].view(np.uint32)
            sc = blob[base + 256 * bits:base + gb].view(np.float16).astype(np.float64)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                if bits == 4:
                    A = [[], []]
                    for h in range(2):
                        w = words[h * 128 + lane * 4: h * 128 + lane * 4 + 4]
                        A[0] += dequant4(int(w[0])) + dequant4(int(w[1]))
                        A[1] += dequant4(int(w[2])) + dequant4(int(w[3]))
                else:
                    w = [int(v) for v in words[lane * 6: lane * 6 + 6]]
                    A = [dequant3(*w[0:3]), dequant3(*w[3:6])]
                for h in range(2):
                    sp = h if d["sets"] == 2 else 0
                    kbase = gi * 128 + 64 * h + 16 * t
                    for hi in range(2):
                        row = sub * 16 + g + 8 * hi
                        wv = np.concatenate(A[hi][8 * h: 8 * h + 8])        # 16 codes i = 0..15
                        y[:, row] += sc[sp * 16 + g + 8 * hi] * (xs[:, kbase:kbase + 16] @ wv)
        for j in range(d["Cp"] // 16):
            o = d["off_cherry"] + sub * d["cher_bytes"] + j * 512
            blk = blob[o:o + 512].view(np.float16).astype(np.float64).reshape(32, 8)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for reg in range(4):
                    row = sub * 16 + g + 8 * (reg & 1)
                    c0 = 16 * j + 2 * t + 8 * (reg >> 1)
                    y[:, row] += xc[:, c0] * blk[lane, 2 * reg] + xc[:, c0 + 1] * blk[lane, 2 * reg + 1]
    return y[:, :N]
