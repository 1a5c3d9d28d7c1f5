"""CPU restatement of PCEngine's kernel-map algorithm (TEST INFRASTRUCTURE ONLY).

This module is the parity checker for the CUDA map-build path.  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may import it; the
product package never does.

PARITY PINNED against the reference's own CUDA code: tests/golden/ref_*.npz hold
what the reference's unmodified extension (compiled by oracle/build_ref.py, run on
a B200 by tests/golden/make_ref_golden.py) returned from ``mapping_d2_cuda`` and
``conv_fwd_d2_cuda`` for submanifold 3x3x3 and strided ks=3 / stride 2 layers, and
tests/test_ref_golden.py checks this file against them bit for bit (output
coordinates, indicator map, knnz, kpos, qkpos).  The reference ships no golden
vectors or known-answer tests of its own.  Forms the reference does not compute
correctly or deterministically (its ks == stride shortcut, odd ks >= 5 strided
layers, atomics-ordered D1 positions) are pinned instead by agreement with dense
``torch.nn.functional.conv3d`` on small grids (tests/test_oracle_dense.py).

Every function cites the reference lines (paths relative to the reference
project root) whose behaviour it restates.  Arithmetic is NumPy int64; nothing
here is written for speed beyond being vectorised over voxels.
"""
from __future__ import annotations

import numpy as np

CODE_X = 94273  # script/utils.py:233-242
CODE_Y = 311
D1_CODE = 1186111  # backend/hash.cuh:7-9 (buffer_encoder)
Q_PAD = 128  # backend/hash.cu:203,430 (q of exclusive_scan_for_kernel_quantified)


def encode3(v) -> int:
    """script/utils.py:233-234 conv_info_encoder."""
    return CODE_X * int(v[0]) + CODE_Y * int(v[1]) + int(v[2])


def decode3(code: int):
    """script/utils.py:237-242 conv_info_decoder (also backend/hash.cu:57-76)."""
    x = code // CODE_X
    y = (code - x * CODE_X) // CODE_Y
    z = code - x * CODE_X - y * CODE_Y
    return (int(x), int(y), int(z))


def mid_index(ks) -> int:
    """Centre weight index, backend/hash.cuh:304-305, backend/spconv.cu:247-248."""
    return (ks[0] - 1) // 2 * ks[1] * ks[2] + (ks[1] - 1) // 2 * ks[2] + (ks[2] - 1) // 2


def kernel_offsets(ks, strided: bool) -> np.ndarray:
    """[kv,3] offsets, kp = (ix*ksy + iy)*ksz + iz with x slowest.

    Submanifold: backend/hash.cuh:313-315 (centred).  Strided: the same plus one
    for odd sizes above one, backend/hash.cuh:396-401 and :585-590.
    """
    ksx, ksy, ksz = ks
    kv = ksx * ksy * ksz
    kp = np.arange(kv)
    kx = kp // (ksz * ksy) - (ksx - 1) // 2
    ky = (kp // ksz) % ksy - (ksy - 1) // 2
    kz = kp % ksz - (ksz - 1) // 2
    if strided:
        kx = kx + (0 if (ksx % 2 == 0 or ksx == 1) else 1)
        ky = ky + (0 if (ksy % 2 == 0 or ksy == 1) else 1)
        kz = kz + (0 if (ksz % 2 == 0 or ksz == 1) else 1)
    return np.stack([kx, ky, kz], axis=1).astype(np.int64)


_BIAS = 1 << 16  # coordinates in [-65536, 65535], batch index below 4096: 3*17 + 12 = 63 bits
_SPAN = 1 << 17


def _pack(b, x, y, z) -> np.ndarray:
    """Order-preserving int64 key of (b,x,y,z); any injective key would do, the
    reference compares a 64-bit mixed hash instead (backend/hash.cuh:11-15)."""
    return ((b.astype(np.int64) * _SPAN + (x + _BIAS)) * _SPAN + (y + _BIAS)) * _SPAN + (z + _BIAS)


class _Table:
    """Exact coordinate -> row lookup (role of insertHash/insertVal + the probe
    loop of the query kernels, backend/hash.cuh:55-91,321-330)."""

    def __init__(self, coords: np.ndarray):
        c = coords.astype(np.int64)
        key = _pack(c[:, 0], c[:, 1], c[:, 2], c[:, 3])
        self.order = np.argsort(key, kind="stable")
        self.keys = key[self.order]

    def find(self, b, x, y, z) -> np.ndarray:
        q = _pack(b, x, y, z)
        if len(self.keys) == 0:
            return np.full(q.shape, -1, np.int64)
        pos = np.searchsorted(self.keys, q)
        pos[pos == len(self.keys)] = 0
        hit = self.keys[pos] == q
        return np.where(hit, self.order[pos], -1)


def _cdiv_trunc(a, b):
    """C integer division (truncation toward zero) on int64 arrays."""
    return (np.abs(a) // b) * np.sign(a)


def strided_output_coords(coords, ks, stride, pad, cmin, cmax) -> np.ndarray:
    """Output coordinates of a strided conv: general ("Expand") rule.

    backend/hash.cuh:535-610 (candidate = in - k + pad, kept when divisible by the
    stride and min <= quotient <= max), then unique and ascending (b,x,y,z)
    (backend/hash.cu:377-396).  ``cmax`` is already the *output* bound computed at
    script/spconv.py:355-360.  The reference's separate ks == stride shortcut
    (backend/hash.cu:333-362) is inconsistent with its own query kernel and is
    not restated; this rule is used for every ks/stride.
    """
    c = coords.astype(np.int64)
    offs = kernel_offsets(ks, True)
    s = np.asarray(stride, np.int64)
    p = np.asarray(pad, np.int64)
    lo = np.asarray(cmin, np.int64)
    hi = np.asarray(cmax, np.int64)
    cand = c[:, None, 1:4] - offs[None, :, :] + p[None, None, :]
    q = _cdiv_trunc(cand, s[None, None, :])
    rem = cand - q * s[None, None, :]
    ok = ((q >= lo) & (q <= hi) & (rem == 0)).all(axis=2)
    b = np.broadcast_to(c[:, None, 0], ok.shape)[ok]
    q = q[ok]
    out = np.concatenate([b[:, None], q], axis=1)
    if len(out) == 0:
        return np.zeros((0, 4), np.int32)
    out = np.unique(out, axis=0)  # lexicographic ascending == ascending linear code
    return out.astype(np.int32)


def indicator_map(in_coords, out_coords, ks, stride, pad, subm: bool) -> np.ndarray:
    """The D2 ("fetch on demand") map: int32 [kv, N_in], map[kp, in_id] = out_id or -1.

    Submanifold: backend/hash.cuh:265-333 (in = out + offset, centre skipped when
    ``separate_mid``; the Python caller passes separate_mid = subm,
    script/spconv.py:362-368).  Strided: backend/hash.cuh:339-419
    (in = out*stride - pad + shifted offset, no centre skipped).
    """
    n_in = len(in_coords)
    kv = ks[0] * ks[1] * ks[2]
    m = np.full((kv, n_in), -1, np.int32)
    if n_in == 0 or len(out_coords) == 0:
        return m
    table = _Table(in_coords)
    oc = out_coords.astype(np.int64)
    offs = kernel_offsets(ks, not subm)
    mid = mid_index(ks)
    if subm:
        base = oc[:, 1:4]
    else:
        base = oc[:, 1:4] * np.asarray(stride, np.int64) - np.asarray(pad, np.int64)
    oid = np.arange(len(oc), dtype=np.int64)
    for kp in range(kv):
        if subm and kp == mid:
            continue
        t = base + offs[kp]
        i = table.find(oc[:, 0], t[:, 0], t[:, 1], t[:, 2])
        hit = i >= 0
        m[kp, i[hit]] = oid[hit]
    return m


def kernel_scans(knnz: np.ndarray):
    """kpos/qkpos, both kv+1 long, backend/hash.cuh:478-497 with q = 128."""
    kv = len(knnz)
    kpos = np.zeros(kv + 1, np.int32)
    qkpos = np.zeros(kv + 1, np.int32)
    kpos[1:] = np.cumsum(knnz)
    qkpos[1:] = np.cumsum((knnz + Q_PAD - 1) // Q_PAD * Q_PAD)
    return kpos, qkpos


def pair_lists(m: np.ndarray):
    """Indicator -> pair lists, ascending (kp, in_id): script/spconv.py:370-372."""
    kv, n_in = m.shape
    flat = m.reshape(-1)
    nz = np.nonzero(flat != -1)[0]
    omap = flat[nz].astype(np.int32)
    imap = (nz % max(n_in, 1)).astype(np.int32)
    kp = (nz // max(n_in, 1)).astype(np.int32)
    return imap, omap, kp


def build_d2(in_coords, ks, stride, pad, cmin, cmax_in, subm: bool) -> dict:
    """Everything ``mapping_d2_cuda`` and the Python post-pass produce.

    ``cmax_in`` is the input tensor's coords_max; the output bound is derived as
    script/spconv.py:355-360 does.  Returns out_coords, map [kv*N_in], knnz, kpos,
    qkpos, imap, omap (pair lists), qsum, cmax_out.
    """
    in_coords = np.ascontiguousarray(in_coords, dtype=np.int32).reshape(-1, 4)
    if subm:
        out_coords = in_coords
        cmax_out = list(cmax_in)
    else:
        cmax_out = [(cmax_in[i] + 2 * pad[i] - (ks[i] - 1)) // stride[i] for i in range(3)]
        out_coords = strided_output_coords(in_coords, ks, stride, pad, cmin, cmax_out)
    m = indicator_map(in_coords, out_coords, ks, stride, pad, subm)
    knnz = (m != -1).sum(axis=1).astype(np.int32)
    kpos, qkpos = kernel_scans(knnz)
    imap, omap, kp = pair_lists(m)
    return dict(out_coords=out_coords, map=m.reshape(-1), knnz=knnz, kpos=kpos, qkpos=qkpos,
                imap=imap, omap=omap, pair_kp=kp, qsum=int(qkpos[-1]), cmax_out=cmax_out,
                n_in=len(in_coords), n_out=len(out_coords), kv=m.shape[0], subm=subm,
                mid=mid_index(ks))


def build_d1(d2: dict) -> dict:
    """The CSR-coded ("gather-mm-scatter") map in canonical form.

    Code = kp*1186111 + pos (backend/hash.cuh:7-9).  The reference draws ``pos``
    from an atomic counter (backend/hash.cuh:161-165) so its value is run
    dependent; the canonical ``pos`` is the pair's index inside its offset's
    segment of the (kp, in_id)-ordered pair list.  Row pointers are the scanned
    per-row hit counts (backend/hash.cuh:422-437, backend/hash.cu:236-243); row
    entries stay kp-ascending because thrust::remove is stable
    (backend/hash.cu:224-231).
    """
    imap, omap, kp = d2["imap"], d2["omap"], d2["pair_kp"]
    kpos = d2["kpos"]
    pidx = np.arange(len(imap), dtype=np.int64)
    code = (kp.astype(np.int64) * D1_CODE + (pidx - kpos[kp])).astype(np.int32)

    def csr(rows, n_rows):
        order = np.lexsort((kp, rows))  # by row, then kp ascending
        ptr = np.zeros(n_rows + 1, np.int32)
        np.add.at(ptr, rows.astype(np.int64) + 1, 1)
        ptr = np.cumsum(ptr).astype(np.int32)
        return ptr, code[order]

    icsr, imap_c = csr(imap, d2["n_in"])
    ocsr, omap_c = csr(omap, d2["n_out"])
    return dict(icsr=icsr, imap=imap_c, ocsr=ocsr, omap=omap_c)


def neighbour_csr(d2: dict, transposed: bool = False) -> dict:
    """Output-major neighbour lists plus the indicator bitmask.

    For every output row: bit kp of ``mask`` is set iff the row has an input at
    offset kp; ``nbr`` lists those inputs kp-ascending; ``rowptr`` delimits rows.
    For a submanifold map the centre offset is included as the identity pair
    (the reference applies it as a separate dense GEMM, backend/spconv.cu:273-298).
    ``transposed`` swaps the roles of the two sides (script/spconv.py:236-244).
    """
    kv = d2["kv"]
    imap, omap, kp = d2["imap"], d2["omap"], d2["pair_kp"]
    n_out, n_in = d2["n_out"], d2["n_in"]
    if d2["subm"]:
        ident = np.arange(n_in, dtype=np.int32)
        imap = np.concatenate([imap, ident])
        omap = np.concatenate([omap, ident])
        kp = np.concatenate([kp, np.full(n_in, d2["mid"], np.int32)])
    if transposed:
        imap, omap = omap, imap
        n_out, n_in = n_in, n_out
    order = np.lexsort((kp, omap))
    rows = omap[order].astype(np.int64)
    rowptr = np.zeros(n_out + 1, np.int64)
    np.add.at(rowptr, rows + 1, 1)
    rowptr = np.cumsum(rowptr).astype(np.int32)
    words = (kv + 31) // 32
    mask = np.zeros((n_out, words), np.uint32)
    k = kp[order].astype(np.int64)
    np.bitwise_or.at(mask, (rows, k // 32), (np.uint32(1) << (k % 32).astype(np.uint32)))
    return dict(mask=mask, rowptr=rowptr, nbr=imap[order].astype(np.int32), n_out=n_out, n_in=n_in)
