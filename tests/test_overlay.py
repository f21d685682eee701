"""The C++ safetensors-overlay writer / reader / family tables against the overlay that the reference's own
requant tool wrote for a tiny seeded checkpoint (tests/golden/overlay_model -> tests/golden/overlay, made by
tests/golden/make_golden.py).  Host-only: the codes come from the CPU oracle here (the GPU test feeds the
same writer from the CUDA quantiser).  Every output file must match byte for byte."""
import json
import os
import struct
import numpy as np
import pytest

import __graft_entry__ as G

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODEL = os.path.join(ROOT, 'tests', 'golden', 'overlay_model')
GOLD = os.path.join(ROOT, 'tests', 'golden', 'overlay')


def read_shard(path):
    with open(path, 'rb') as f:
        n = struct.unpack('<Q', f.read(8))[0]
        hdr = json.loads(f.read(n))
        blob = f.read()
    return hdr, blob


def selected_tensors(P, arch='glm5', families=None):
    """(name, bf16 bits [N,K]) in the order the reference tool visits them: shards sorted, header order."""
    for sh in sorted(f for f in os.listdir(MODEL) if f.endswith('.safetensors')):
        hdr, blob = read_shard(os.path.join(MODEL, sh))
        for name, t in hdr.items():
            if name == '__metadata__' or t['dtype'] != 'BF16' or len(t['shape']) != 2 or t['shape'][1] % 16:
                continue
            if P.overlay_family(arch, families, name) < 0:
                continue
            o0, o1 = t['data_offsets']
            yield name, np.frombuffer(blob[o0:o1], np.uint16).reshape(t['shape'])


def write_overlay(P, out, quantise):
    w = P.OverlayWriter(out, shard_bytes=12000)
    n = 0
    for name, bits in selected_tensors(P):
        p, s, gs = quantise(bits)
        w.add(name, p, s, float(gs[0])); n += 1
    w.close()
    return n


def assert_same_files(out):
    names = sorted(os.listdir(GOLD))
    assert sorted(os.listdir(out)) == names
    for f in names:
        assert open(os.path.join(out, f), 'rb').read() == open(os.path.join(GOLD, f), 'rb').read(), f


def test_family_tables():
    P = G.load_package()
    fam = P.overlay_family
    assert fam('glm5', None, 'model.layers.0.self_attn.q_proj.weight') == 0          # kda_qkv, first of the default list
    assert fam('glm5', None, 'lm_head.weight') == 2
    assert fam('glm5', None, 'model.layers.3.self_attn.index_kpool_compress_gate') == 5
    assert fam('glm5', None, 'model.layers.0.mlp.gate.weight') == -1                  # the router stays bf16
    assert fam('glm5', None, 'model.layers.1.self_attn.kv_b_proj.weight') == -1
    assert fam('glm5', None, 'model.visual.layers.0.self_attn.o_proj.weight') == -1   # vision tower excluded
    assert fam('glm5', None, 'visual.blocks.0.self_attn.o_proj.weight') == -1
    assert fam('glm5', None, 'model.embed_tokens.weight') == -1
    assert fam('glm5', 'o_proj,lm_head', 'model.layers.0.self_attn.q_proj.weight') == -1
    assert fam('glm5', 'o_proj, lm_head', 'lm_head.weight') == 1
    assert fam('glm5', 'nonsense', 'lm_head.weight') == -2 and fam('other', None, 'lm_head.weight') == -2
    # the second table is anchored: an audio tower's o_proj must not match
    assert fam('mimo', None, 'model.layers.7.self_attn.o_proj.weight') == 0
    assert fam('mimo', None, 'audio_encoder.input_local_transformer.layers.0.self_attn.o_proj.weight') == -1
    assert fam('mimo', None, 'model.mtp.layers.0.self_attn.o_proj.weight') == -1
    assert fam('mimo', 'o_proj,mtp_o', 'model.mtp.layers.0.self_attn.o_proj.weight') == 1


def test_writer_is_byte_identical_to_the_reference_tool(tmp_path):
    P, O = G.load_package(), G.load_oracle()
    out = str(tmp_path / 'ov')
    n = write_overlay(P, out, lambda bits: O.quantize_tensor(O.bf16_bits_to_f32(bits)))
    assert n == 7
    assert_same_files(out)


def test_reader_round_trip(tmp_path):
    P, O = G.load_package(), G.load_oracle()
    ov = P.Overlay(GOLD)
    try:
        assert len(ov) == 7
        for name, bits in selected_tensors(P):
            p, s, gs, aligned = ov.triple(name)
            rp, rs, rgs = O.quantize_tensor(O.bf16_bits_to_f32(bits))
            assert np.array_equal(p, rp) and np.array_equal(s, rs) and gs.view(np.uint32)[0] == rgs.view(np.uint32)[0], name
            assert aligned, name                      # every tensor of an overlay sits on a 16-byte boundary
        with pytest.raises(P.B200Error):
            ov.triple('model.layers.0.mlp.gate.weight')
    finally:
        ov.close()
    with pytest.raises(P.B200Error):
        P.Overlay(str(tmp_path / 'missing'))


@pytest.mark.gpu
def test_gpu_quantiser_feeds_the_writer_byte_identically(tmp_path):
    import torch
    P = G.load_package()
    out = str(tmp_path / 'ov_gpu')

    def on_gpu(bits):
        W = P.quantize(torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16))
        return W.numpy()
    write_overlay(P, out, on_gpu)
    assert_same_files(out)
