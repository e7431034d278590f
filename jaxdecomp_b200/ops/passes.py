"""Compile a step list (:mod:`.plan`) into tile passes for the native kernels.

Each run ``[Fft] [A2A] [Perm ...]`` of a step list becomes one pass: a strided
read of the local block, an optional 1-D transform along one axis, and a
scatter whose addresses already include the all-to-all routing (which peer,
which chunk) and every local permutation that follows.  The compilation is
pure integer arithmetic on shapes, so it is unit-tested without a GPU and
without a process group; the CPU emulation in the native module executes the
same descriptors with the buffers of all emulated ranks in one process.

Roles of the three local axes in a pass (see ``csrc/tile_map.h``):
``c`` transform axis (copy passes: the input-contiguous axis), ``t`` the axis
tiled together with ``c``, ``o`` the remaining axis.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

from .plan import A2A, Fft, Perm, Step


def _contig_strides(shape: Sequence[int]) -> List[int]:
    st, acc = [0] * len(shape), 1
    for i in range(len(shape) - 1, -1, -1):
        st[i] = acc
        acc *= int(shape[i])
    return st


def _is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


@dataclass
class PassSpec:
    """Geometry of one pass, independent of dtype and of buffer addresses."""

    in_shape: Tuple[int, int, int]
    out_shape: Tuple[int, int, int]
    axes: Tuple[int, int, int]          # local axis playing the role (c, t, o)
    ext: Tuple[int, int, int]           # (C, Tn, On)
    in_strides: Tuple[int, int, int]    # (is_c, is_t, is_o)
    out_strides: Tuple[int, int, int]   # (os_c, os_t, os_o)
    chunks: Tuple[int, int, int]        # (Cl, Tl, Ol)
    out_base: int
    npeers: int
    fft: bool
    mesh_axis: Optional[int]            # decomposition axis of the all-to-all, if any
    plain: bool = False                 # same strides in and out, single destination: may run in place
    concat_role: Optional[int] = None   # role (0 c, 1 t, 2 o) of the axis the all-to-all concatenates along

    @property
    def numel(self) -> int:
        return self.in_shape[0] * self.in_shape[1] * self.in_shape[2]


@dataclass
class _Group:
    fft_axis: Optional[int] = None
    a2a: Optional[A2A] = None
    perms: List[Perm] = field(default_factory=list)


def _group_steps(steps: Sequence[Step], pdims: Sequence[int]) -> List[_Group]:
    groups: List[_Group] = []
    cur: Optional[_Group] = None

    def close():
        nonlocal cur
        if cur is not None and (cur.fft_axis is not None or cur.a2a is not None or cur.perms):
            groups.append(cur)
        cur = None

    for st in steps:
        if isinstance(st, Fft):
            close()
            cur = _Group(fft_axis=st.axis)
        elif isinstance(st, A2A):
            if int(pdims[st.mesh_axis]) == 1:
                continue  # all-to-all over a single rank is the identity
            if cur is None or cur.a2a is not None or cur.perms:
                close()
                cur = _Group()
            cur.a2a = st
        elif isinstance(st, Perm):
            if cur is None:
                cur = _Group()
            cur.perms.append(st)
        else:  # pragma: no cover
            raise TypeError(st)
    close()
    return groups


def compile_passes(steps: Sequence[Step], local_shape: Sequence[int], pdims: Sequence[int],
                   coords: Sequence[int]) -> Tuple[List[PassSpec], Tuple[int, int, int]]:
    """Return the passes for one rank and the local shape of the result."""
    shape = [int(s) for s in local_shape]
    passes: List[PassSpec] = []
    for g in _group_steps(steps, pdims):
        S = list(shape)
        in_st = _contig_strides(S)
        S1 = list(S)
        P, r, split, concat, maxis = 1, 0, None, None, None
        if g.a2a is not None:
            maxis = g.a2a.mesh_axis
            P, r = int(pdims[maxis]), int(coords[maxis])
            split, concat = g.a2a.split, g.a2a.concat
            if S[split] % P:
                raise ValueError(f"local extent {S[split]} of axis {split} cannot be split over {P} ranks")
            S1[split] //= P
            S1[concat] *= P
        order = [0, 1, 2]
        for pm in g.perms:
            order = [order[i] for i in pm.order]
        F = [S1[order[i]] for i in range(3)]
        fs = _contig_strides(F)
        out_st = [0, 0, 0]
        for i, d in enumerate(order):
            out_st[d] = fs[i]
        chunk = [S[d] // P if d == split else S[d] for d in range(3)]
        out_base = r * S[concat] * out_st[concat] if g.a2a is not None else 0

        in_contig = 2  # local blocks are always dense, last axis fastest
        out_contig = order[2]
        if g.fft_axis is not None:
            c = g.fft_axis
            others = [d for d in range(3) if d != c]
            if out_contig != c:
                t = out_contig
            elif in_contig != c:
                t = in_contig
            else:
                t = max(others)  # the faster-varying of the two remaining axes
            if in_contig not in (c, t) or out_contig not in (c, t):
                raise NotImplementedError(
                    f"pass with transform axis {c} reads contiguously along {in_contig} and writes along "
                    f"{out_contig}: needs a three-axis tile"
                )
        else:
            c = in_contig
            if out_contig != c:
                t = out_contig
            else:
                t = max(d for d in range(3) if d != c)
        o = [d for d in range(3) if d not in (c, t)][0]
        roles = (c, t, o)
        spec = PassSpec(
            in_shape=tuple(S), out_shape=tuple(F), axes=roles,
            ext=tuple(S[d] for d in roles),
            in_strides=tuple(in_st[d] for d in roles),
            out_strides=tuple(out_st[d] for d in roles),
            chunks=tuple(chunk[d] for d in roles),
            out_base=out_base, npeers=P, fft=g.fft_axis is not None, mesh_axis=maxis,
        )
        spec.plain = P == 1 and tuple(spec.in_strides) == tuple(spec.out_strides)
        if g.a2a is not None:
            spec.concat_role = roles.index(concat)
        passes.append(spec)
        shape = F
    return passes, tuple(shape)


# ---- pipelining of an exchange pass with the local pass that consumes it -------------------------------------

def pipeline_cut(prod: PassSpec, cons: PassSpec, want_chunks: int) -> Optional[Tuple[int, int, int]]:
    """How to cut an exchange pass and the local pass after it into matching chunks.

    Returns ``(producer role, consumer role, chunks)`` with roles numbered as in the native
    descriptor (2 = t, 3 = o), or ``None`` when the pair cannot be pipelined.  The cut runs along an
    axis of the exchanged array that

    * is neither the producer's transform/split axis nor the axis its all-to-all concatenates along
      (every source rank then contributes to every chunk, and chunk k of all sources together is
      exactly the part of the array with that axis in chunk k),
    * is not the consumer's transform axis (the consumer needs whole rows of that one),

    so that chunk k of the consumer reads only what chunk k of the producers wrote.  The chunk count
    is the largest ``want_chunks / 2**i >= 2`` that divides the extent into whole tiles (ranges along a
    ``t`` axis must be multiples of 32 rows, the largest tile height).
    """
    if prod.npeers <= 1 or cons.npeers != 1 or tuple(prod.out_shape) != tuple(cons.in_shape) or want_chunks < 2:
        return None
    for pr in (2, 1):
        if prod.chunks[pr] != prod.ext[pr] or prod.concat_role == pr or prod.ext[pr] < 2:
            continue
        for cr in (2, 1):
            if cons.in_strides[cr] != prod.out_strides[pr] or cons.ext[cr] != prod.ext[pr]:
                continue
            ext = prod.ext[pr]
            k = int(want_chunks)
            while k >= 2:
                ok = ext % k == 0
                if ok and (pr == 1 or cr == 1):
                    ok = (ext // k) % 32 == 0
                if ok:
                    return pr + 1, cr + 1, k
                k //= 2
    return None


# ---- dtype-dependent tiling ----------------------------------------------------------------------------------

def _env_int(name: str) -> Optional[int]:
    v = os.environ.get(name)
    return int(v) if v not in (None, "") else None


def _log2(n: int) -> int:
    return int(n).bit_length() - 1


def mixed_radix_ok(n: int, elem_bytes: int) -> bool:
    """True when a transform of length ``n`` can use the mixed-radix kernel: prime factors up to 13 and
    two padded rows within the shared memory of one block (``JD_B200_MIXED=0`` forces Bluestein)."""
    if os.environ.get("JD_B200_MIXED", "1") == "0" or n < 2:
        return False
    m = n
    stages = 0
    twos = 0
    while m % 2 == 0:
        m //= 2
        twos += 1
    stages += (twos + 3) // 4
    for p in (3, 5, 7, 11, 13):
        while m % p == 0:
            m //= p
            stages += 1
    if m != 1 or stages > 12:
        return False
    rowlen = n + 2 * ((n + 15) // 16) + 16
    return 2 * rowlen * elem_bytes <= 220 * 1024


def choose_tiling(spec: PassSpec, elem_bytes: int, remote: bool) -> dict:
    """Pick the tile extents, shared-memory pitch and access-width flags."""
    C, Tn, On = spec.ext
    is_c, is_t, is_o = spec.in_strides
    os_c, os_t, os_o = spec.out_strides
    Cl, Tl, Ol = spec.chunks
    load_t = is_c != 1
    store_t = os_c != 1
    out = {"load_t_contig": int(load_t), "store_t_contig": int(store_t)}
    out["split_axis"] = 1 if Cl != C else (2 if Tl != Tn else (3 if Ol != On else 0))
    intra_pad = 0
    if spec.fft and not (_is_pow2(C) and C >= 8) and mixed_radix_ok(C, elem_bytes):
        # mixed-radix kernel: two shared-memory buffers of T padded rows
        rowlen = C + 2 * ((C + 15) // 16)
        lanes = 16 if elem_bytes == 8 else 8  # elements per shared-memory wavefront
        pitch = rowlen + (lanes // 8 - rowlen) % lanes
        tile_bytes = lambda t: 2 * t * pitch * elem_bytes  # noqa: E731
        T = 1
        while T < 32 and tile_bytes(2 * T) <= 110 * 1024:
            T *= 2
        if store_t:
            # stored runs of at least 64 bytes, at the price of one resident block per SM
            while T * elem_bytes < 64 and tile_bytes(2 * T) <= 220 * 1024:
                T *= 2
        T = min(T, _next_pow2(Tn))
        ov = _env_int("JD_B200_TILE_T")
        if ov:
            T = max(1, min(_next_pow2(ov), 32))
            while T > 1 and tile_bytes(T) > 220 * 1024:
                T //= 2
        # the last stage of a rotating pass reads min(T, 8) rows x lanes / min(T, 8) columns per wavefront:
        # conflict-free when the pitch equals that column count modulo the wavefront width
        pitch = rowlen + (lanes // min(T, 8) - rowlen) % lanes
        out.update(fft_mode=3, M=C, T=T, Cc=C, pitch=pitch, logW=_log2(_next_pow2(C)))
        intra_pad = 1
    elif spec.fft:
        pow2 = _is_pow2(C) and C >= 8
        M = C if pow2 else max(8, _next_pow2(2 * C - 1))
        out["fft_mode"] = 1 if pow2 else 2
        out["M"] = M
        if M > 16384 * 8 // elem_bytes:
            raise NotImplementedError(f"transform length {C} needs {M} points of shared memory; not supported")
        if M >= 128 and os.environ.get("JD_B200_INTRAPAD", "1") != "0":
            intra_pad = 1
        rowlen = M + (M >> 3) if intra_pad else M
        target = 80 * 1024
        T = 1
        while T < 32 and (2 * T) * rowlen * elem_bytes <= target and (2 * T) * M * elem_bytes <= 16384 * 8:
            T *= 2
        T = min(T, _next_pow2(Tn))
        ov = _env_int("JD_B200_TILE_T")
        if ov:
            T = max(1, min(_next_pow2(ov), 32))
            while T > 1 and (T * M * elem_bytes > 16384 * 8 or T * (rowlen + 4) * elem_bytes > 220 * 1024):
                T //= 2
        rp = _env_int("JD_B200_ROWPAD")
        if rp is not None:
            pad = rp
        elif not (load_t or store_t):
            pad = 0
        elif elem_bytes == 8:
            pad = max(2, 32 // T)
            pad += pad & 1
        else:
            pad = max(1, 16 // T)
        out["T"] = T
        out["Cc"] = M
        out["pitch"] = rowlen + pad
        out["logW"] = _log2(M)
    else:
        out["fft_mode"] = 0
        out["M"] = 0
        Cc = _env_int("JD_B200_COPY_CC") or (64 if elem_bytes <= 8 else 32)
        Cc = min(_next_pow2(Cc), _next_pow2(C))
        T = min(_next_pow2(_env_int("JD_B200_COPY_T") or 32), _next_pow2(Tn))
        pad = {4: 1, 8: 2, 16: 1}[elem_bytes] if (load_t or store_t) and T > 1 else 0
        if _env_int("JD_B200_COPY_PAD") is not None and pad:
            pad = _env_int("JD_B200_COPY_PAD")
        out["T"] = T
        out["Cc"] = Cc
        out["pitch"] = Cc + pad
        out["logW"] = _log2(Cc)
    T = out["T"]
    out["logT"] = _log2(T)
    out["intra_pad"] = intra_pad
    vec_in = vec_out = 0
    if elem_bytes == 8 and out["pitch"] % 2 == 0:
        even = lambda *v: all(int(x) % 2 == 0 for x in v)  # noqa: E731
        if load_t:
            vec_in = int(T % 2 == 0 and even(Tn, is_c, is_o))
        else:
            vec_in = int(even(C, is_t, is_o) and (spec.fft or out["Cc"] % 2 == 0))
        if store_t:
            vec_out = int(T % 2 == 0 and even(Tn, Tl, os_c, os_o, spec.out_base))
        else:
            vec_out = int(even(C, Cl, os_t, os_o, spec.out_base) and (spec.fft or out["Cc"] % 2 == 0))
    out["vec_in"], out["vec_out"] = vec_in, vec_out
    bulk = 0
    if spec.fft and out["fft_mode"] == 1 and not load_t and not intra_pad and os.environ.get("JD_B200_BULK", "1") != "0":
        if (C * elem_bytes) % 16 == 0 and (is_t * elem_bytes) % 16 == 0 and (is_o * elem_bytes) % 16 == 0 \
                and (out["pitch"] * elem_bytes) % 16 == 0:
            bulk = 1
    out["use_bulk"] = bulk
    return out


def check_pass_bounds(spec: PassSpec) -> None:
    """Index-range check done once, when a plan is built: the largest element offset a pass can read
    or write must stay inside the dense block of ``numel`` elements on either side.  (The kernels
    themselves carry no per-access checks; every address they form is one of the offsets bounded here.)"""
    ext = spec.ext
    hi_in = sum((e - 1) * s for e, s in zip(ext, spec.in_strides))
    hi_out = spec.out_base + sum((c - 1) * s for c, s in zip(spec.chunks, spec.out_strides))
    lo_out = spec.out_base
    if hi_in >= spec.numel or lo_out < 0 or hi_out >= spec.numel:
        raise AssertionError(
            f"tile pass addresses leave the block: max input offset {hi_in}, output offsets [{lo_out}, {hi_out}], "
            f"block of {spec.numel} elements ({spec})"
        )


def fill_desc(native, spec: PassSpec, elem_bytes: int, inverse: bool, scale: float, batch: int,
              remote: bool, device_tables: bool):
    """Build a native ``PassDesc`` (addresses left empty) for a pass."""
    check_pass_bounds(spec)
    d = native.PassDesc()
    C, Tn, On = spec.ext
    d.C, d.Tn, d.On, d.B = C, Tn, On, int(batch)
    d.is_c, d.is_t, d.is_o = spec.in_strides
    d.os_c, d.os_t, d.os_o = spec.out_strides
    d.is_b = spec.numel
    d.os_b = spec.numel
    d.Cl, d.Tl, d.Ol = spec.chunks
    d.out_base = spec.out_base
    d.out_limit = spec.numel * int(batch)
    d.npeers = spec.npeers
    d.elem_bytes = elem_bytes
    d.inverse = int(bool(inverse)) if spec.fft else 0
    d.scale = float(scale) if spec.fft else 1.0
    tl = choose_tiling(spec, elem_bytes, remote)
    for k, v in tl.items():
        setattr(d, k, v)
    if spec.fft:
        tw, ch, bh, tws = native.get_fft_tables(C, tl["M"], elem_bytes, device_tables)
        d.twiddle, d.chirp, d.bhat, d.tw_stage = tw, ch, bh, tws
    return d
