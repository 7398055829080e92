"""Weights from a safetensors file: header parsing on the CPU (no device), and on a GPU the on-load quantisation,
whose packed bytes must equal quantising the same fp32 tensor in one piece (the oracle's bytes)."""
import json
import struct

import numpy as np
import pytest

import oracle as o
import ullm_cuda as U
from ullm_cuda import _abi as abi


def write_safetensors(path, tensors, metadata=None):
    """tensors: {name: (dtype string, shape, raw bytes)} -> the public safetensors container format."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def test_header_parsing_needs_no_device(tmp_path):
    w = np.arange(6 * 256, dtype=np.float32).reshape(6, 256)
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, {"a.weight": ("F32", w.shape, w.tobytes()),
                          "b \"quoted\"": ("BF16", (4, 128), bytes(4 * 128 * 2)),
                          "vec": ("F16", (128,), bytes(256)),
                          "codes": ("F8_E4M3", (2, 16), bytes(32))},
                      metadata={"format": "pt", "note": "nested {\"x\": [1, 2]}"})
    info = U.safetensors_find(p, "a.weight")
    assert (info.dtype, info.rank, info.rows, info.cols, info.data_bytes) == (abi.DTYPE_F32, 2, 6, 256, w.nbytes)
    with open(p, "rb") as f:
        f.seek(info.data_offset)
        assert f.read(16) == w.tobytes()[:16]
    info = U.safetensors_find(p, 'b "quoted"')
    assert (info.dtype, info.rows, info.cols) == (abi.DTYPE_BF16, 4, 128)
    info = U.safetensors_find(p, "vec")
    assert (info.dtype, info.rank, info.rows, info.cols) == (abi.DTYPE_F16, 1, 1, 128)
    for name, status in (("missing", U.Status.InvalidArgument), ("codes", U.Status.Unsupported)):
        with pytest.raises(U.CudaError) as e:
            U.safetensors_find(p, name)
        assert e.value.status is status, e.value
    assert "e4m3fn" in e.value.message  # 8-bit float payloads are never reinterpreted
    bad = str(tmp_path / "bad.safetensors")
    with open(bad, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(U.CudaError) as e:
        U.safetensors_find(bad, "x")
    assert e.value.status is U.Status.InvalidArgument
    lying = str(tmp_path / "lying.safetensors")
    write_safetensors(lying, {"w": ("F32", (4, 128), bytes(100))})  # offsets do not match the shape
    with pytest.raises(U.CudaError) as e:
        U.safetensors_find(lying, "w")
    assert e.value.status is U.Status.InvalidArgument
    with pytest.raises(U.CudaError):
        U.safetensors_find(str(tmp_path / "nope.safetensors"), "w")


@pytest.mark.gpu
@pytest.mark.parametrize("encoding", [U.ENCODING_AQ4, U.ENCODING_FP8_CHANNEL])
@pytest.mark.parametrize("src", ["F32", "BF16", "F16"])
def test_quantise_at_load_equals_one_piece_quantisation(gpu, tmp_path, encoding, src):
    ctx, q = gpu
    n, k = 1500, 4096  # 24 MB of fp32: more than one 16 MiB staging chunk
    w = o.planted_case_weights(o.DEFAULT_SEED, 6100, n, k)
    if src == "F32":
        raw, wq = w.tobytes(), w
    elif src == "BF16":
        bits = o.f32_to_bf16_bits(w)
        raw, wq = bits.tobytes(), o.bf16_bits_to_f32(bits).reshape(n, k)
    else:
        h = w.astype(np.float16)
        raw, wq = h.tobytes(), h.astype(np.float32)
    p = str(tmp_path / "w.safetensors")
    write_safetensors(p, {"other": ("F32", (2, 2), bytes(16)), "layer.0.w": (src, (n, k), raw)}, metadata={"format": "pt"})
    vb, sb = U.weight_bytes(encoding, n, k)
    vals, scl = ctx.alloc(vb + 256), ctx.alloc(sb + 256)
    q.fill(vals.at(0), 0xC5, vb + 256)
    q.fill(scl.at(0), 0xC5, sb + 256)
    wd = U.weight_desc(encoding, n, k, vals.at(0), scl.at(0))
    q.quantize_safetensors(p, "layer.0.w", wd)
    if encoding == U.ENCODING_AQ4:
        v, s = o.aq4_quantize(wq)
        assert np.array_equal(q.download(vals.at(0), (n, k // 2), np.uint8), v)
        assert np.array_equal(q.download(scl.at(0), (n, k // 128), np.float16).view(np.uint16), s.view(np.uint16))
    else:
        v, s = o.fp8_quantize(wq)
        assert np.array_equal(q.download(vals.at(0), (n, k), np.uint8), v)
        assert np.array_equal(q.download(scl.at(0), (n,), np.float32).view(np.uint32), s.view(np.uint32))
    assert (q.download(vals.at(vb), (256,), np.uint8) == 0xC5).all() and (q.download(scl.at(sb), (256,), np.uint8) == 0xC5).all()
    with pytest.raises(U.CudaError) as e:  # the descriptor must state the stored shape
        q.quantize_safetensors(p, "layer.0.w", U.weight_desc(encoding, n, k // 2, vals.at(0), scl.at(0)))
    assert e.value.status is U.Status.InvalidArgument
    vals.close()
    scl.close()
