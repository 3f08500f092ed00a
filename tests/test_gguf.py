"""The GGUF reader against files written here from synthetic layers: the tensors it
hands over are the bytes that went in (separate and fused gate/up tensors, quantised
and float types), the layer it builds gives the oracle the same result, and broken
files are refused."""
import struct

import numpy as np
import pytest

import oracle
from biv_b200 import workloads as W
from biv_b200.gguf import GgufError, GgufFile, T_STR, T_U32, T_U64


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, layer, block=3, fused=False, arch="qwen35moe", align=32, version=3):
    """A GGUF file holding one block's MoE tensors (and a decoy tensor in front)."""
    kv = [("general.architecture", T_STR, arch), ("general.alignment", T_U32, align),
          (f"{arch}.embedding_length", T_U64, layer.n_embd), (f"{arch}.expert_count", T_U64, layer.n_expert),
          (f"{arch}.expert_used_count", T_U64, layer.n_expert_used),
          (f"{arch}.expert_feed_forward_length", T_U64, layer.n_ff_exp),
          (f"{arch}.expert_shared_feed_forward_length", T_U64, layer.n_ff_shexp if layer.has_shared else 0),
          ("tokenizer.ggml.scores", 9, np.arange(5, dtype=np.float32))]
    p = f"blk.{block}."

    def whole(st):      # the stack's matrices, back to back
        return np.concatenate([st.expert(i) for i in range(st.n)])
    tensors = [("token_embd.weight", 0, [4, 2], np.zeros(32, np.uint8)),
               (p + "ffn_gate_inp.weight", 0, [layer.n_embd, layer.n_expert],
                np.ascontiguousarray(layer.router, np.float32).view(np.uint8).reshape(-1))]
    e, ff, n = layer.n_embd, layer.n_ff_exp, layer.n_expert
    if fused:
        both = np.concatenate([np.concatenate([layer.gate.expert(i), layer.up.expert(i)]) for i in range(n)])
        tensors.append((p + "ffn_gate_up_exps.weight", layer.gate.ty, [e, 2 * ff, n], both))
    else:
        tensors.append((p + "ffn_gate_exps.weight", layer.gate.ty, [e, ff, n], whole(layer.gate)))
        tensors.append((p + "ffn_up_exps.weight", layer.up.ty, [e, ff, n], whole(layer.up)))
    tensors.append((p + "ffn_down_exps.weight", layer.down.ty, [ff, e, n], whole(layer.down)))
    if layer.has_shared:
        sff = layer.n_ff_shexp
        tensors += [(p + "ffn_gate_shexp.weight", layer.sh_gate.ty, [e, sff], whole(layer.sh_gate)),
                    (p + "ffn_up_shexp.weight", layer.sh_up.ty, [e, sff], whole(layer.sh_up)),
                    (p + "ffn_down_shexp.weight", layer.sh_down.ty, [sff, e], whole(layer.sh_down)),
                    (p + "ffn_gate_inp_shexp.weight", 0, [e],
                     np.ascontiguousarray(layer.sh_gate_inp, np.float32).view(np.uint8).reshape(-1))]
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv))
    for key, ty, val in kv:
        head += _s(key) + struct.pack("<I", ty)
        if ty == T_STR:
            head += _s(val)
        elif ty == T_U32:
            head += struct.pack("<I", val)
        elif ty == T_U64:
            head += struct.pack("<Q", val)
        else:   # an array of f32
            head += struct.pack("<IQ", 6, len(val)) + val.tobytes()
    off, infos, blobs = 0, b"", []
    for name, ty, dims, data in tensors:
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ty, off)
        pad = -len(data) % align
        blobs.append(data.tobytes() + b"\0" * pad)
        off += len(data) + pad
    body = head + infos
    body += b"\0" * (-len(body) % align)
    with open(path, "wb") as f:
        f.write(body + b"".join(blobs))


@pytest.mark.parametrize("cfg,fused", [("parity_q8_0", False), ("decode_q4k", True), ("ep_bf16", False)])
def test_layer_read_back_from_a_file(tmp_path, cfg, fused):
    wl = getattr(W, cfg)(n=6, **W.SMALL)
    layer = wl.layers[0]
    path = tmp_path / "m.gguf"
    write_gguf(path, layer, block=3, fused=fused)
    g = GgufFile(str(path))
    try:
        got = g.moe_layer(3)
        assert (got.n_embd, got.n_expert, got.n_expert_used, got.n_ff_exp) == \
            (layer.n_embd, layer.n_expert, layer.n_expert_used, layer.n_ff_exp)
        for a, b in ((got.gate, layer.gate), (got.up, layer.up), (got.down, layer.down),
                     (got.sh_gate, layer.sh_gate), (got.sh_down, layer.sh_down)):
            assert a.ty == b.ty and (a.cols, a.rows, a.n) == (b.cols, b.rows, b.n)
            for i in range(a.n):
                np.testing.assert_array_equal(a.expert(i), b.expert(i))
        if fused:       # one tensor, two views: same bytes, the up rows half a matrix further
            assert got.gate.data.ctypes.data == got.up.data.ctypes.data and got.up.offset > 0
        np.testing.assert_array_equal(got.router, layer.router)
        np.testing.assert_array_equal(oracle.moe_forward(got, wl.h), oracle.moe_forward(layer, wl.h))
    finally:
        g.close()


@pytest.mark.parametrize("gate_ty,down_ty", [(W.Q4_0, W.Q4_1), (W.F16, W.F32)])
def test_the_other_tensor_types_read_back(tmp_path, gate_ty, down_ty):
    wl = W.typed_layer(gate_ty, down_ty, n=4, **W.SMALL)
    layer = wl.layers[0]
    path = tmp_path / "m.gguf"
    write_gguf(path, layer, block=1, fused=True)
    g = GgufFile(str(path))
    try:
        got = g.moe_layer(1)
        assert (got.gate.ty, got.down.ty) == (gate_ty, down_ty)
        np.testing.assert_array_equal(oracle.moe_forward(got, wl.h), oracle.moe_forward(layer, wl.h))
    finally:
        g.close()


def test_broken_files_are_refused(tmp_path):
    wl = W.parity_q8_0(n=2, **W.SMALL)
    path = tmp_path / "m.gguf"
    (tmp_path / "junk").write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(GgufError):
        GgufFile(str(tmp_path / "junk"))
    write_gguf(path, wl.layers[0], arch="llama")
    g = GgufFile(str(path))
    with pytest.raises(GgufError):
        g.moe_layer(3)
    g.close()
    write_gguf(path, wl.layers[0])
    g = GgufFile(str(path))
    with pytest.raises(GgufError):          # no such block
        g.moe_layer(4)
    g.close()
    data = path.read_bytes()
    (tmp_path / "cut.gguf").write_bytes(data[:len(data) // 2])
    g = GgufFile(str(tmp_path / "cut.gguf"))
    with pytest.raises(GgufError):          # a tensor runs past the end of the file
        g.moe_layer(3)
    g.close()


@pytest.mark.gpu
def test_layer_from_a_file_on_the_gpu(tmp_path):
    import torch
    from biv_b200.moe import Moe
    from helpers import rel_err
    wl = W.decode_q4k(n=20, **W.SMALL)
    path = tmp_path / "m.gguf"
    write_gguf(path, wl.layers[0], block=0, fused=True)
    g = GgufFile(str(path))
    layer = g.moe_layer(0)
    m = Moe(layer, wl.n)            # the fused tensor goes in as two views with one stride
    try:
        out = m.moe(torch.from_numpy(wl.h).cuda()).cpu().numpy()
    finally:
        m.close()
        g.close()
    assert rel_err(out, oracle.moe_forward(wl.layers[0], wl.h)) < 1e-3
