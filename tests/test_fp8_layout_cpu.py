"""The index arithmetic of the e4m3 converter warps of attn_decode_tc.cu, restated and
checked on the CPU: which piece of a raw tile a lane takes, where it lands in the fp16
operand tile, and that the eight lanes of a 16-byte access never share a bank group.

Layouts (both under the 128-byte swizzle: 16-byte chunk c of row r sits at
r * 128 + ((c ^ (r % 8)) << 4)):
  raw K / V tile   [128 keys][128 e4m3 bytes]
  fp16 K tile      [2 halves of 64 head_dim][128 keys][128 B]       (K-major: head_dim along a row)
  fp16 V tile      [2 halves of 64 keys][128 head_dim rows][128 B]  (transposed: keys along a row)
"""

import numpy as np

HALF = 128 * 128


def swz(row, chunk):
    return row * 128 + ((chunk ^ (row & 7)) << 4)


def raw_tile(ids):
    """Shared-memory image (one id per byte) of a raw tile whose byte (key, b) is ids[key, b]."""
    img = np.full(128 * 128, -1, dtype=np.int64)
    for key in range(128):
        for c in range(8):
            img[swz(key, c): swz(key, c) + 16] = ids[key, 16 * c: 16 * c + 16]
    return img


def bank_groups(addresses):
    return {(a >> 4) & 7 for a in addresses}


def test_k_pieces_cover_the_tile_without_bank_conflicts():
    ids = np.arange(128 * 128, dtype=np.int64).reshape(128, 128)   # id = key * 128 + head_dim
    raw = raw_tile(ids)
    out = np.full(2 * HALF // 2, -1, dtype=np.int64)                # one slot per fp16 element
    for cw in range(4):                                             # the K quartet
        for n in range(8):
            loads, stores0, stores1 = [], [], []
            for lane in range(32):
                row = 8 * cw + (lane & 7) + 32 * (n >> 1)
                col = (lane >> 3) + 4 * (n & 1)                     # 16-byte column of the raw row
                src = swz(row, col)
                ch = 2 * (lane >> 3)                                # fp16 chunks ch, ch + 1 of half n % 2
                at = (n & 1) * HALF
                d0, d1 = at + swz(row, ch), at + swz(row, ch + 1)
                loads.append(src), stores0.append(d0), stores1.append(d1)
                piece = raw[src: src + 16]
                out[d0 >> 1: (d0 >> 1) + 8] = piece[:8]
                out[d1 >> 1: (d1 >> 1) + 8] = piece[8:]
            for q in range(4):                                      # a 16-byte access goes eight lanes at a time
                for acc in (loads, stores0, stores1):
                    assert len(bank_groups(acc[8 * q: 8 * q + 8])) == 8
    for key in range(128):
        for hd in range(128):
            at = (hd // 64) * HALF + swz(key, (hd % 64) // 8) + (hd % 8) * 2
            assert out[at >> 1] == ids[key, hd]


def test_v_pieces_are_transposed_without_bank_conflicts():
    ids = np.arange(128 * 128, dtype=np.int64).reshape(128, 128)
    raw = raw_tile(ids)
    out = np.full(2 * HALF // 2, -1, dtype=np.int64)
    for cw in range(4):                                             # the V quartet
        for n in range(8):
            kb = 4 * cw + (n >> 1)                                  # block of eight keys
            # ldmatrix.x4: lane 8 m + i gives the address of row i of matrix m
            addr = [swz(8 * kb + (lane & 7), 4 * (n & 1) + (lane >> 3)) for lane in range(32)]
            for m in range(4):
                assert len(bank_groups(addr[8 * m: 8 * m + 8])) == 8
            # thread t receives bytes 4 (t % 4) .. + 3 of row t / 4 of every matrix
            w = np.zeros((32, 4, 4), dtype=np.int64)
            for t in range(32):
                for m in range(4):
                    a = addr[8 * m + t // 4] + 4 * (t % 4)
                    w[t, m] = raw[a: a + 4]
            at = (kb >> 3) * HALF
            for which in range(2):                                  # the two stmatrix.x4.trans
                for m in range(4):
                    rows = []
                    for i in range(8):                              # lane 8 m + i addresses row i of matrix m
                        pair = i >> 1
                        hd_x = 4 * pair + 2 * (pair >> 1) + (i & 1)
                        hd_y = 4 * pair + 2 * (1 - (pair >> 1)) + (i & 1)
                        hd = 16 * (4 * (n & 1) + m) + (hd_x if which == 0 else hd_y)
                        a = at + swz(hd, kb & 7)
                        rows.append(a)
                        for key in range(8):                        # memory row i = M[i][0..7], M[2 (t % 4) + e][t / 4] from thread t
                            t, e = key * 4 + pair, i & 1
                            swap = (t & 2) != 0
                            lo, hi = w[t, m, 0:2], w[t, m, 2:4]
                            reg = (hi if swap else lo) if which == 0 else (lo if swap else hi)
                            out[(a >> 1) + key] = reg[e]
                    assert len(bank_groups(rows)) == 8
    for hd in range(128):
        for key in range(128):
            at = (key // 64) * HALF + swz(hd, (key % 64) // 8) + (key % 8) * 2
            assert out[at >> 1] == ids[key, hd]


def test_integer_route_of_the_conversion_is_exact():
    """A byte s.eeee.mmm in the top half of a 16-bit lane, shifted right by one under its
    sign, times 2^8: the fp16 value of every e4m3 byte that is not NaN."""
    from oracle import attention_oracle as orc
    values = orc.e4m3_values()
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        x = b << 8
        bits = ((x >> 1) & 0x3F80) | (x & 0x8000)
        got = float(np.array([bits], dtype=np.uint16).view(np.float16)[0]) * 256.0
        assert got == float(values[b]), (b, got, values[b])
