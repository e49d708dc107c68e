"""Generates the golden fixtures in this directory from the UNMODIFIED reference.

Run where the reference checkout and its shim are available:

    make -C oracle ref && python tests/golden/generate.py

Every case seeds poisoned owner storage plus a seeded logical payload, runs one
operation through the reference CPU backend's own DeviceOps facade (portable
build; BF16 RMSNorm additionally through the AVX-512 BF16 build) and records
the inputs' and the result's complete physical (tiled) storage. The fixtures
are small (a few KB each) and are committed; the GPU box has no reference
checkout and checks against these files.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

from iom_b200.tensor import DataType  # noqa: E402
from support import Reference, SPECIAL_BF16, SPECIAL_F32, random_payload  # noqa: E402

POISON = 0xA5


def owner(ref, shape, dtype, payload):
    tensor = ref.tensor(shape, dtype)
    tensor.storage[:] = POISON
    tensor.view().from_host(payload)
    return tensor


def transformed(view, steps):
    for name, args in steps:
        view = getattr(view, name)(*args)
    return view


def describe(view):
    dims, offset, strides, _ = view.describe()
    return np.array(list(dims) + [offset] + list(strides), dtype=np.int64)


def binary_cases(ref, out):
    shapes = [((2, 17, 33), (2, 17, 33), (2, 17, 33)), ((2, 1, 33), (1, 17, 1), (2, 17, 33)),
              ((32, 48), (1, 48), (32, 48)), ((32, 48), (32, 1), (32, 48)),
              ((5, 31), (1, 1), (5, 31))]
    for dtype in (DataType.I32, DataType.F32, DataType.BF16):
        for op, code in (("add", 0), ("mul", 1), ("sub", 2), ("div", 3)):
            if op == "div" and dtype == DataType.I32:
                continue      # the reference admits no integer division
            for i, (ls, rs, os_) in enumerate(shapes):
                rng = np.random.default_rng(1000 + 10 * int(dtype) + i)
                lhs = owner(ref, ls, dtype, random_payload(rng, ls, dtype))
                rhs = owner(ref, rs, dtype, random_payload(rng, rs, dtype))
                res = owner(ref, os_, dtype, random_payload(rng, os_, dtype))
                before = res.storage.copy()
                token = ref.lib.iomref_binary(ref.queue, code, lhs.view().handle, rhs.view().handle,
                                              res.view().handle)
                assert ref.run(token) == 0, ref.error()
                key = f"binary_{op}_{dtype.name}_{i}"
                out[key + "_lhs"] = lhs.storage.copy()
                out[key + "_rhs"] = rhs.storage.copy()
                out[key + "_out_before"] = before
                out[key + "_out"] = res.storage.copy()
                out[key + "_shapes"] = np.array([len(ls), *ls, len(rs), *rs, len(os_), *os_])
    for dtype, specials in ((DataType.F32, SPECIAL_F32), (DataType.BF16, SPECIAL_BF16)):
        n = len(specials)
        for op, code in (("add", 0), ("mul", 1), ("sub", 2), ("div", 3)):
            lhs = owner(ref, (n, n), dtype, np.repeat(specials, n).reshape(n, n))
            rhs = owner(ref, (n, n), dtype, np.tile(specials, n).reshape(n, n))
            res = owner(ref, (n, n), dtype, np.zeros((n, n), dtype=specials.dtype))
            token = ref.lib.iomref_binary(ref.queue, code, lhs.view().handle, rhs.view().handle,
                                          res.view().handle)
            assert ref.run(token) == 0
            key = f"special_{op}_{dtype.name}"
            out[key + "_lhs"] = lhs.storage.copy()
            out[key + "_rhs"] = rhs.storage.copy()
            out[key + "_out"] = res.storage.copy()


SMALL_FLOATS = ((DataType.F8_E4M3FN, 8), (DataType.F8_E5M2, 8), (DataType.F6_E2M3, 6),
                (DataType.F6_E3M2, 6), (DataType.F4_E2M1, 4))


def pack_codes(codes, bits):
    """LSB-first bit stream of `codes` (the logical host form of a leaf narrower than a byte)."""
    flat = np.asarray(codes, dtype=np.uint64).reshape(-1)
    stream = np.zeros((flat.size * bits + 7) // 8, dtype=np.uint8)
    for k in range(bits):
        position = np.arange(flat.size, dtype=np.uint64) * bits + k
        bit = ((flat >> np.uint64(k)) & np.uint64(1)).astype(np.uint8)
        np.bitwise_or.at(stream, (position >> np.uint64(3)).astype(np.int64), bit << (position & np.uint64(7)).astype(np.uint8))
    return stream


def every_pair_cases(ref, out):
    """All pairs of codes of the 8-, 6- and 4-bit floating leaves, four operations each: an
    [N, N] tensor with N = 2^bits, lhs[i, j] = i, rhs[i, j] = j."""
    for dtype, bits in SMALL_FLOATS:
        n = 1 << bits
        codes = np.arange(n, dtype=np.uint8)
        first, second = np.repeat(codes, n), np.tile(codes, n)
        if bits < 8:
            first, second = pack_codes(first, bits), pack_codes(second, bits)
        zeros = np.zeros_like(first)
        for op, code in (("add", 0), ("mul", 1), ("sub", 2), ("div", 3)):
            lhs, rhs, res = owner(ref, (n, n), dtype, first), owner(ref, (n, n), dtype, second), \
                owner(ref, (n, n), dtype, zeros)
            token = ref.lib.iomref_binary(ref.queue, code, lhs.view().handle, rhs.view().handle,
                                          res.view().handle)
            assert ref.run(token) == 0, ref.error()
            key = f"pairs_{op}_{dtype.name}"
            out[key + "_lhs"] = lhs.storage.copy()
            out[key + "_rhs"] = rhs.storage.copy()
            out[key + "_out"] = res.storage.copy()


def rmsnorm_cases(ref, out, tag):
    for dtype in (DataType.BF16, DataType.F32):
        for i, shape in enumerate([(1, 1), (15, 17), (17, 33), (2, 3, 16, 31), (4, 256), (18, 1040)]):
            rng = np.random.default_rng(2000 + 10 * int(dtype) + i)
            x = owner(ref, shape, dtype, random_payload(rng, shape, dtype, "normal"))
            w = owner(ref, (1, shape[-1]), dtype, random_payload(rng, (1, shape[-1]), dtype, "normal"))
            res = owner(ref, shape, dtype, random_payload(rng, shape, dtype))
            before = res.storage.copy()
            token = ref.lib.iomref_rmsnorm(ref.queue, x.view().handle, w.view().handle,
                                           res.view().handle, 1e-5)
            assert ref.run(token) == 0, ref.error()
            key = f"rmsnorm_{tag}_{dtype.name}_{i}"
            out[key + "_x"] = x.storage.copy()
            out[key + "_w"] = w.storage.copy()
            out[key + "_out_before"] = before
            out[key + "_out"] = res.storage.copy()
            out[key + "_shape"] = np.array(shape)


def mover_cases(ref, out):
    rng = np.random.default_rng(3000)
    src = owner(ref, (3, 4, 17, 33), DataType.BF16, random_payload(rng, (3, 4, 17, 33), DataType.BF16))
    dst = owner(ref, (4, 3, 17, 33), DataType.BF16, random_payload(rng, (4, 3, 17, 33), DataType.BF16))
    out["copy_dst_before"] = dst.storage.copy()
    sv = transformed(src.view(), [("slice", (1, 0, 2, 2))])
    dv = transformed(dst.view(), [("permute", ([1, 0],)), ("slice", (1, 1, 2, 2))])
    assert ref.run(ref.lib.iomref_copy(ref.queue, sv.handle, dv.handle)) == 0
    out["copy_src"] = src.storage.copy()
    out["copy_dst"] = dst.storage.copy()
    out["copy_src_view"] = describe(sv)
    out["copy_dst_view"] = describe(dv)

    table = owner(ref, (50, 37), DataType.BF16, random_payload(rng, (50, 37), DataType.BF16))
    ids = rng.integers(0, 50, size=(2, 1, 19)).astype(np.uint32)
    idx = owner(ref, (2, 1, 19), DataType.U32, ids)
    res = owner(ref, (2, 19, 37), DataType.BF16, random_payload(rng, (2, 19, 37), DataType.BF16))
    out["embedding_out_before"] = res.storage.copy()
    assert ref.run(ref.lib.iomref_embedding(ref.queue, table.view().handle, idx.view().handle,
                                            res.view().handle)) == 0
    out["embedding_table"] = table.storage.copy()
    out["embedding_ids"] = idx.storage.copy()
    out["embedding_out"] = res.storage.copy()

    for a in (0, 5, 29):
        s = owner(ref, (2, 3, 3, 40), DataType.BF16, random_payload(rng, (2, 3, 3, 40), DataType.BF16))
        d = owner(ref, (2, 3, 32, 40), DataType.BF16, random_payload(rng, (2, 3, 32, 40), DataType.BF16))
        out[f"append_{a}_dst_before"] = d.storage.copy()
        assert ref.run(ref.lib.iomref_cache_append(ref.queue, s.view().handle, d.view().handle, a)) == 0
        out[f"append_{a}_src"] = s.storage.copy()
        out[f"append_{a}_dst"] = d.storage.copy()

    # host transfer: logical payload -> tiled storage of a transformed view
    host = owner(ref, (3, 2, 17, 35), DataType.F32, random_payload(rng, (3, 2, 17, 35), DataType.F32))
    out["transfer_before"] = host.storage.copy()
    view = transformed(host.view(), [("permute", ([1, 0],)), ("slice", (1, 1, 2, 1))])
    payload = random_payload(rng, (2, 2, 17, 35), DataType.F32)
    view.from_host(payload)
    out["transfer_payload"] = payload
    out["transfer_after"] = host.storage.copy()
    out["transfer_view"] = describe(view)


def silu_cases(ref, out, tag):
    """SiLU through the reference CPU backend (FP32 evaluation, expf of this host's
    C library): every BF16 code, and a ragged multi-plane F32 case with specials."""
    codes = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    x = owner(ref, (256, 256), DataType.BF16, codes)
    y = owner(ref, (256, 256), DataType.BF16, np.zeros((256, 256), dtype=np.uint16))
    assert ref.run(ref.lib.iomref_silu(ref.queue, x.view().handle, y.view().handle)) == 0, ref.error()
    out[f"silu_{tag}_BF16_out"] = y.storage.copy()
    rng = np.random.default_rng(4000)
    payload = (random_payload(rng, (2, 17, 35), DataType.F32, "normal") * np.float32(6.0)).astype(np.float32)
    flat = payload.reshape(-1).view(np.uint32)
    flat[:SPECIAL_F32.size] = SPECIAL_F32
    xf = owner(ref, (2, 17, 35), DataType.F32, payload)
    yf = owner(ref, (2, 17, 35), DataType.F32, random_payload(rng, (2, 17, 35), DataType.F32))
    out[f"silu_{tag}_F32_out_before"] = yf.storage.copy()
    assert ref.run(ref.lib.iomref_silu(ref.queue, xf.view().handle, yf.view().handle)) == 0, ref.error()
    out[f"silu_{tag}_F32_x"] = xf.storage.copy()
    out[f"silu_{tag}_F32_out"] = yf.storage.copy()


ROPE_CASES = [((2, 3, 5, 64), 0, 10000.0), ((4, 17, 128), 7, 10000.0), ((1, 2, 33, 34), 2040, 500000.0)]


def rope_cases(ref, out, tag):
    """RoPE through the reference CPU backend (FP32 carrier; powf / sinf / cosf of this
    host's C library fix the angle bits)."""
    for dtype in (DataType.BF16, DataType.F32):
        for i, (shape, a, theta) in enumerate(ROPE_CASES):
            rng = np.random.default_rng(5000 + 10 * int(dtype) + i)
            x = owner(ref, shape, dtype, random_payload(rng, shape, dtype, "normal"))
            y = owner(ref, shape, dtype, random_payload(rng, shape, dtype))
            key = f"rope_{tag}_{dtype.name}_{i}"
            out[key + "_out_before"] = y.storage.copy()
            token = ref.lib.iomref_rope(ref.queue, x.view().handle, y.view().handle, a, theta)
            assert ref.run(token) == 0, ref.error()
            out[key + "_x"] = x.storage.copy()
            out[key + "_out"] = y.storage.copy()


def main():
    fixtures = {}
    portable = Reference("portable")
    binary_cases(portable, fixtures)
    rmsnorm_cases(portable, fixtures, "portable")
    mover_cases(portable, fixtures)
    silu_cases(portable, fixtures, "portable")
    rope_cases(portable, fixtures, "portable")
    every_pair_cases(portable, fixtures)
    portable.close()
    avx = Reference("avx512")
    assert avx.lib.iomref_avx512_bf16_active() == 1, "this host cannot run the AVX-512 BF16 build"
    rmsnorm_cases(avx, fixtures, "avx512")
    silu_cases(avx, fixtures, "avx512")
    rope_cases(avx, fixtures, "avx512")
    avx.close()
    np.savez_compressed(HERE / "reference_vectors.npz", **fixtures)
    print(f"wrote {len(fixtures)} arrays, "
          f"{(HERE / 'reference_vectors.npz').stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
