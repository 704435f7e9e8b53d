"""numpy statement of the fragment layout (test infrastructure): the expected bytes of
rb200_preprocess_weight for a matrix of unsigned codes.  Written from the layout description in
relax_b200/csrc/dequant.cuh, independently of the CUDA repack kernel."""
import numpy as np


def unit_pos(lane: int) -> int:
    """16-byte unit position of lane 4g+t inside a 512-byte tile: 8t + ((g + 2t) & 7)."""
    g, t = lane >> 2, lane & 3
    return 8 * t + ((g + 2 * t) & 7)


def _place_units(tiles: np.ndarray) -> np.ndarray:
    """tiles[..., lane, unit payload] -> same shape with lane's unit moved to unit_pos(lane)."""
    out = np.empty_like(tiles)
    for lane in range(32):
        out[..., unit_pos(lane), :] = tiles[..., lane, :]
    return out


def tile_offset(nb: int, kb: int, NB: int, KB: int) -> int:
    """Byte offset of fragment tile (nb, kb): tiles of one (128-row tile, 4-k-block chunk) are contiguous."""
    t, b, c, j = nb // 8, nb % 8, kb // 4, kb % 4
    nblk = min(8, NB - 8 * t)
    nkb = min(4, KB - 4 * c)
    return ((t * 8 * KB) + c * 4 * nblk + b * nkb + j) * 512


def _order_tiles(tiles: np.ndarray) -> np.ndarray:
    """tiles uint8 [NB, KB, 512] -> flat bytes in storage order."""
    NB, KB, _ = tiles.shape
    out = np.empty(NB * KB * 512, dtype=np.uint8)
    seen = np.zeros(NB * KB, dtype=bool)
    for nb in range(NB):
        for kb in range(KB):
            o = tile_offset(nb, kb, NB, KB)
            assert o % 512 == 0 and not seen[o // 512]
            seen[o // 512] = True
            out[o:o + 512] = tiles[nb, kb]
    assert seen.all()
    return out


def fragment_layout(codes: np.ndarray, bits: int) -> np.ndarray:
    """codes uint8 [N, K] (unsigned) -> uint8 flat array of N*K*bits/8 bytes."""
    n, k = codes.shape
    if bits == 4:
        kb = k // 64
        # [nb, r2, g, kb, t, j, c] with n = nb*16 + r2*8 + g, k = kb*64 + t*16 + j*4 + c
        c = codes.reshape(n // 16, 2, 8, kb, 4, 4, 4).astype(np.uint32)
        # nibble slot p for (r2, c): c=0 -> p=0/1, c=1 -> p=4/5, c=2 -> p=2/3, c=3 -> p=6/7
        slot = np.array([[0, 4, 2, 6], [1, 5, 3, 7]])
        words = np.zeros((n // 16, 8, kb, 4, 4), dtype=np.uint32)  # [nb, g, kb, t, j]
        for r2 in range(2):
            for cc in range(4):
                words |= c[:, r2, :, :, :, :, cc] << np.uint32(4 * slot[r2, cc])
        # memory order: nb, kb, unit position of lane (g, t), j
        tiles = words.transpose(0, 2, 1, 3, 4).reshape(n // 16, kb, 32, 4)  # [nb, kb, lane=4g+t, j]
        return _order_tiles(_place_units(tiles).astype("<u4").view(np.uint8).reshape(n // 16, kb, 512))
    kb = k // 32
    # [nb, r2, g, kb, t, j, c] with k = kb*32 + t*8 + j*4 + c
    c = codes.reshape(n // 16, 2, 8, kb, 4, 2, 4)
    # memory order: nb, kb, unit position of lane (g, t), then (j, r2, c) inside the 16-byte unit
    tiles = np.ascontiguousarray(c.transpose(0, 3, 2, 4, 5, 1, 6)).reshape(n // 16, kb, 32, 16)
    return _order_tiles(_place_units(tiles).astype(np.uint8).reshape(n // 16, kb, 512))
