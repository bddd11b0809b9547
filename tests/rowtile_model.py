"""Numpy model of the row-tile layout (cq_rlayer in include/cherryq.h): builds the device blob of a
layer from the reference-format buffers, byte for byte, and decodes it again.  Test infrastructure:
the GPU re-pack kernel is compared with `build_blob`, and `decode_codes` walks the blob the way the
one-row decode kernel's lanes do (same masks, same shifts), so the documented layout, the re-pack
and the kernel's unpack are pinned against each other."""
import numpy as np

from oracle import cherryq_oracle as O


def dims(bits, K, N, Cn, G):
    Kc = K - Cn
    NG = (Kc + 127) // 128
    sets = 2 if G == 64 else 1
    Cp = (Cn + 15) // 16 * 16
    NT = (N + 15) // 16
    tile_bytes = NG * 256 * bits + NG * sets * 32 + Cp // 16 * 512
    al = lambda v: (v + 255) // 256 * 256
    off_tiles = 0
    off_perm = al(NT * tile_bytes)
    off_cidx = al(off_perm + NG * 128 * 2)
    off_work = al(off_cidx + max(Cp, 16) * 2)
    ksplit = (NG + 63) // 64           # layers of more than 64 groups carry a work area for their column parts
    blob_bytes = off_work if ksplit == 1 else al(off_work + ksplit * NT * 16 * 4 * 4 + NT * 4)
    return dict(bits=bits, K=K, N=N, C=Cn, G=G, Kc=Kc, NG=NG, sets=sets, Cp=Cp, NT=NT, tile_bytes=tile_bytes,
                ksplit=ksplit, off_work=off_work,
                scal_off=NG * 256 * bits, cher_off=NG * 256 * bits + NG * sets * 32, off_tiles=off_tiles,
                off_perm=off_perm, off_cidx=off_cidx, blob_bytes=blob_bytes)


def _word_offset3(lane, widx):
    return lane * 16 + widx * 4 if widx < 4 else 512 + lane * 8 + (widx - 4) * 4


def build_blob(qweight, scales, cherry_weight, cherry_indices, bits, K, G):
    N = qweight.shape[1]
    Cn = len(cherry_indices)
    d = dims(bits, K, N, Cn, G)
    u = O.unpack_codes(qweight, bits).astype(np.uint32)              # (Kc, N) unsigned codes
    rows = d["NT"] * 16
    codes = np.zeros((d["NG"] * 128, rows), dtype=np.uint32)
    codes[:d["Kc"], :N] = u
    blob = np.zeros(d["blob_bytes"], dtype=np.uint8)
    tiles = np.zeros((d["NT"], d["tile_bytes"] // 4), dtype=np.uint32)
    gw = 64 * bits                                                     # words per group block
    lane = np.arange(32)
    g8, t = lane >> 2, lane & 3
    for gg in range(d["NG"]):
        c = codes[gg * 128:(gg + 1) * 128].reshape(128, d["NT"], 16)  # [column][tile][row in tile]

        def reg(chunk, j):
            """A-fragment register j of a 32-column chunk for every (tile, lane): 4 codes as [tile][lane][b]."""
            rl = g8 + 8 * (j & 1)
            kb = 32 * chunk + 16 * (j >> 1) + 4 * t
            cols = kb[:, None] + np.arange(4)[None, :]                 # (lane, b)
            return c[cols, :, rl[:, None]].transpose(2, 0, 1)          # (tile, lane, b)

        def bytes_to_word(v):                                          # (tile, lane, 4 bytes) -> (tile, lane)
            return v[..., 0] | (v[..., 1] << 8) | (v[..., 2] << 16) | (v[..., 3] << 24)

        base = gg * gw
        if bits == 4:
            for l in range(2):
                for j in range(4):
                    w = bytes_to_word(reg(2 * l, j) | (reg(2 * l + 1, j) << 4))
                    idx = base + (l * 512 + lane * 16 + j * 4) // 4
                    tiles[:, idx] = w
        else:
            for s in range(2):
                r3p, r3h = reg(2 * s, 3), reg(2 * s + 1, 3)
                for wi in range(3):
                    v = reg(2 * s, wi) | (reg(2 * s + 1, wi) << 4) | (((r3p >> wi) & 1) << 3) | (((r3h >> wi) & 1) << 7)
                    w = bytes_to_word(v)
                    offs = np.array([_word_offset3(int(ln), 3 * s + wi) for ln in lane])
                    tiles[:, base + offs // 4] = w
    tb = tiles.view(np.uint8).reshape(d["NT"], d["tile_bytes"])
    # scales [group][set][g8][row g8, row g8 + 8]
    sc = np.zeros((d["NT"], d["NG"] * d["sets"], 8, 2), dtype=np.float16)
    ngr = (d["Kc"] + G - 1) // G
    for gs in range(d["NG"] * d["sets"]):
        kc = (gs // d["sets"]) * 128 + (gs % d["sets"]) * 64
        gi = kc // G
        if kc < d["Kc"] and gi < ngr:
            full = np.zeros(rows, dtype=np.float16)
            full[:N] = scales[gi]
            sc[:, gs] = full.reshape(d["NT"], 2, 8).transpose(0, 2, 1)
    tb[:, d["scal_off"]:d["cher_off"]] = sc.view(np.uint8).reshape(d["NT"], -1)
    # cherry A fragments
    if d["Cp"]:
        cw = np.zeros((d["Cp"], rows), dtype=np.float16)
        cw[:Cn, :N] = cherry_weight
        ch = np.zeros((d["NT"], d["Cp"] // 16, 32, 4, 2), dtype=np.float16)
        for cc in range(16):
            for rl in range(16):
                ln = (rl & 7) * 4 + ((cc & 7) >> 1)
                j = ((cc >> 3) << 1) | (rl >> 3)
                vals = cw[cc::16].reshape(d["Cp"] // 16, d["NT"], 16)[:, :, rl]      # (block, tile)
                ch[:, :, ln, j, cc & 1] = vals.T
        tb[:, d["cher_off"]:] = ch.view(np.uint8).reshape(d["NT"], -1)
    blob[:d["NT"] * d["tile_bytes"]] = tb.reshape(-1)
    perm = np.full(d["NG"] * 128, K, dtype=np.uint16)
    perm[:d["Kc"]] = O.normal_columns(K, np.asarray(cherry_indices, dtype=np.int64)).astype(np.uint16)
    blob[d["off_perm"]:d["off_perm"] + perm.nbytes] = perm.view(np.uint8)
    cidx = np.full(max(d["Cp"], 0), K, dtype=np.uint16)
    cidx[:Cn] = np.asarray(cherry_indices).astype(np.uint16)
    blob[d["off_cidx"]:d["off_cidx"] + cidx.nbytes] = cidx.view(np.uint8)
    return blob, d


def decode_codes(blob, d):
    """The codes as the kernel's lanes see them: masks and shifts of the MMA unpack, (Kc, N)."""
    bits = d["bits"]
    tb = blob[:d["NT"] * d["tile_bytes"]].reshape(d["NT"], d["tile_bytes"])
    out = np.zeros((d["NG"] * 128, d["NT"] * 16), dtype=np.uint32)
    lane = np.arange(32)
    g8, t = lane >> 2, lane & 3
    for gg in range(d["NG"]):
        words = tb[:, gg * 256 * bits:(gg + 1) * 256 * bits].copy().view(np.uint32)       # (tile, words)

        def put(chunk, j, reg, mult):
            """reg: (tile, lane) words holding four u8 = mult * code."""
            for b in range(4):
                v = ((reg >> (8 * b)) & 0xFF) // mult
                rl = g8 + 8 * (j & 1)
                col = gg * 128 + 32 * chunk + 16 * (j >> 1) + 4 * t + b
                for ln in range(32):
                    out[col[ln], np.arange(d["NT"]) * 16 + rl[ln]] = v[:, ln]

        if bits == 4:
            for l in range(2):
                for j in range(4):
                    w = words[:, (l * 512 + lane * 16 + j * 4) // 4]
                    put(2 * l, j, w & 0x0F0F0F0F, 1)
                    put(2 * l + 1, j, w & 0xF0F0F0F0, 16)
        else:
            for s in range(2):
                A, B, Cw = (words[:, np.array([_word_offset3(int(ln), 3 * s + wi) for ln in lane]) // 4] for wi in range(3))
                A3, B2, C1 = A >> 3, B >> 2, Cw >> 1
                for j, w in enumerate((A, B, Cw)):
                    put(2 * s, j, w & 0x07070707, 1)
                    put(2 * s + 1, j, w & 0x70707070, 16)
                put(2 * s, 3, (A3 & 0x01010101) | (B2 & 0x02020202) | (C1 & 0x04040404), 1)
                put(2 * s + 1, 3, (A3 & 0x10101010) | (B2 & 0x20202020) | (C1 & 0x40404040), 16)
    return out[:d["Kc"], :d["N"]]
