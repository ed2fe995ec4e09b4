"""CPU-only checks of the C ABI: the library loads, exports what the header declares, the struct layouts agree,
the integer bucket table is bit-exact against the HuggingFace fixtures, and argument errors are reported before any
launch."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from flashdeberta_b200 import _lib, bucket
from flashdeberta_b200.attention import lengths_from_mask
from tests._golden import load_bucket_golden

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fdb_b200.h")


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.load()
    text = open(HEADER).read()
    declared = set(re.findall(r"FDB_API[^;(]*?\b(fdb_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found in the header"
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fdb_abi_version() == _lib.ABI_VERSION


def test_struct_layout_matches_the_header(tmp_path):
    fields = [f[0] for f in _lib.AttnParams._fields_]
    src = tmp_path / "layout.c"
    body = "\n".join(f'  printf("{f} %zu\\n", offsetof(fdb_attn_params, {f}));' for f in fields)
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "fdb_b200.h"\nint main(void) {\n'
        '  printf("sizeof %zu\\n", sizeof(fdb_attn_params));\n' + body + "\n  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = dict(line.split() for line in subprocess.check_output([str(exe)], text=True).splitlines())
    assert int(out["sizeof"]) == C.sizeof(_lib.AttnParams)
    for f in fields:
        assert int(out[f]) == getattr(_lib.AttnParams, f).offset, f


def test_backward_block_layout_matches_the_header(tmp_path):
    from flashdeberta_b200 import backward
    fields = [f[0] for f in backward.BwdBlock._fields_]
    src = tmp_path / "layout_bwd.c"
    body = "\n".join(f'  printf("{f} %zu\\n", offsetof(fdb_bwd_block, {f}));' for f in fields)
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "fdb_b200.h"\nint main(void) {\n'
        '  printf("sizeof %zu\\n", sizeof(fdb_bwd_block));\n' + body + "\n  return 0;\n}\n")
    exe = tmp_path / "layout_bwd"
    subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    out = dict(line.split() for line in subprocess.check_output([str(exe)], text=True).splitlines())
    assert int(out["sizeof"]) == C.sizeof(backward.BwdBlock)
    for f in fields:
        assert int(out[f]) == getattr(backward.BwdBlock, f).offset, f


def test_backward_block_argument_errors():
    from flashdeberta_b200 import backward
    lib = _lib.load()
    p = backward.BwdBlock()
    assert lib.fdb_attn_bwd_probs(C.byref(p), None) == -1          # struct_bytes missing
    p.struct_bytes = C.sizeof(backward.BwdBlock)
    p.groups, p.heads, p.seqlen, p.row0, p.rows = 6, 4, 128, 0, 64  # groups not a multiple of heads
    assert lib.fdb_attn_bwd_probs(C.byref(p), None) == -1
    p.groups = 8
    p.row0 = 100                                                     # block reaches past the sequence
    assert lib.fdb_attn_bwd_probs(C.byref(p), None) == -1
    p.row0 = 0
    assert lib.fdb_attn_bwd_probs(C.byref(p), None) == -1          # tensors missing
    assert lib.fdb_attn_bwd_bucket_sums(C.byref(p), None) == -1    # no tables, no dscores
    assert lib.fdb_last_error().decode() != ""
    p.rows = 0
    p.scores = p.dprobs = p.lse = p.delta = p.probs = p.dscores = 0x1000
    assert lib.fdb_attn_bwd_probs(C.byref(p), None) == 0           # an empty block is a no-op


def _configs(g):
    for k in g:
        if k.startswith("idx_"):
            _, b, m = k.split("_")
            yield int(b), int(m)


def test_bucket_table_bit_exact_vs_hf_fixture():
    g = load_bucket_golden()
    d_lo, d_hi = int(g["d_lo"]), int(g["d_hi"])
    for buckets, max_rel in _configs(g):
        want = g[f"idx_{buckets}_{max_rel}"].astype(np.int64)
        tab, d_min = bucket.host_lut(buckets, max_rel)
        d = np.arange(d_lo, d_hi + 1)
        got = tab[np.clip(d - d_min, 0, len(tab) - 1)].astype(np.int64)
        assert np.array_equal(got, want), (buckets, max_rel)
        # the saturation claim: first/last entries hold beyond the table
        assert tab[0] == want[0] and tab[-1] == want[-1]
        for dist in (-40000, -513, -512, -129, -1, 0, 1, 128, 129, 505, 506, 40000):
            assert bucket.relative_index(dist, buckets, max_rel) == want[dist - d_lo]


def test_v3_table_shape():
    tab, d_min = bucket.host_lut(256, 512)
    assert (len(tab), d_min, int(tab[0]), int(tab[-1])) == (1019, -512, 0, 511)
    assert np.all(np.diff(tab.astype(np.int32)) >= 0)


def _params(**kw):
    p = _lib.AttnParams()
    p.struct_bytes = C.sizeof(_lib.AttnParams)
    p.dtype = _lib.FDB_BF16
    p.q = p.k = p.v = p.out = 0x1000
    for n in ("q", "k", "v"):
        setattr(p, n + "_row_stride", 128)
        setattr(p, n + "_head_stride", 64)
    p.out_row_stride, p.out_head_stride = 128, 64
    p.batch, p.max_seqlen, p.total_rows, p.heads, p.head_dim = 2, 64, 128, 2, 64
    p.sm_scale = 0.125
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("change,code", [
    (dict(struct_bytes=8), -1),
    (dict(q=0), -1),
    (dict(head_dim=128), -2),
    (dict(dtype=_lib.FDB_FP32), -2),
    (dict(dtype=7), -1),
    (dict(q=0x1008), -3),
    (dict(q_row_stride=130), -3),
    (dict(total_rows=100), -1),
    (dict(sm_scale=0.0), -1),
    (dict(pos_key=0x2000), -1),       # tables without a bucket table
    (dict(seq_lens=0x10, cu_seqlens=0x10), -1),
    (dict(prepared=4), -1),           # unknown bit
])
def test_argument_errors_are_reported_before_any_launch(change, code):
    lib = _lib.load()
    p = _params(**change)
    assert lib.fdb_attn_fwd(C.byref(p), None) == code
    assert lib.fdb_last_error().decode() != ""
    with pytest.raises(_lib.FdbError):
        _lib.check(lib.fdb_attn_fwd(C.byref(p), None))


def test_missing_workspace_is_an_error():
    lib = _lib.load()
    p = _params()
    need = lib.fdb_attn_workspace_bytes(C.byref(p))
    assert need > 0 and need % 256 == 0
    assert lib.fdb_attn_fwd(C.byref(p), None) == -4


def test_lengths_from_every_mask_form():
    m2 = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [0, 0, 0, 0]])
    want = [3, 1, 0]
    assert lengths_from_mask(m2).tolist() == want
    ext = m2.unsqueeze(1).unsqueeze(2)
    m4 = ext * ext.squeeze(-2).unsqueeze(-1)
    assert lengths_from_mask(m4).tolist() == want
    assert lengths_from_mask(m4[:, 0]).tolist() == want
    assert lengths_from_mask(torch.tensor(want)).tolist() == want
    assert lengths_from_mask(None) is None


def test_ops_refuse_cpu_tensors():
    from flashdeberta_b200 import ops
    x = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.disentangled_attention(x, x, x, None, None, max_seqlen=8)


@pytest.mark.parametrize("x,gamma,hidden,code", [
    (0, 0x1000, 768, -1),          # x NULL
    (0x1000, 0, 768, -1),          # gamma NULL
    (0x1000, 0x1000, 100, -2),     # hidden not a multiple of 256
    (0x1000, 0x1000, 4096, -2),    # hidden above 2048
    (0x1008, 0x1000, 768, -3),     # x not 16-byte aligned
])
def test_add_layernorm_argument_errors(x, gamma, hidden, code):
    lib = _lib.load()
    rc = lib.fdb_add_layernorm(x or None, None, gamma or None, 0x1000, 0x2000, 4, hidden, 1e-7, None)
    assert rc == code
    assert lib.fdb_last_error().decode() != ""


def test_add_layernorm_zero_rows_is_a_no_op():
    lib = _lib.load()
    assert lib.fdb_add_layernorm(0x1000, None, 0x1000, 0x1000, 0x2000, 0, 768, 1e-7, None) == 0


def test_layer_output_blocks_keep_transformers_parameter_names():
    """The blocks that call the fused add + LayerNorm are drop-in for transformers' (same state-dict keys), and fall back to
    transformers' own expression on CPU tensors."""
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Layer
    from flashdeberta_b200.model import FlashDebertaV2Layer
    cfg = DebertaV2Config(hidden_size=256, num_attention_heads=4, intermediate_size=512, num_hidden_layers=1,
                          relative_attention=True, position_buckets=32, max_relative_positions=64,
                          pos_att_type="c2p|p2c", share_att_key=True, vocab_size=100, type_vocab_size=0)
    cfg.attn_backend = "b200"
    torch.manual_seed(0)
    ours, theirs = FlashDebertaV2Layer(cfg).eval(), DebertaV2Layer(cfg).eval()
    assert set(ours.state_dict().keys()) == set(theirs.state_dict().keys())
    theirs.load_state_dict(ours.state_dict())
    h, x = torch.randn(2, 5, 512), torch.randn(2, 5, 256)
    with torch.no_grad():
        assert torch.equal(ours.output(h, x), theirs.output(h, x))
        assert torch.equal(ours.attention.output(x, x), theirs.attention.output(x, x))
        assert torch.equal(ours.intermediate(x), theirs.intermediate(x))


@pytest.mark.parametrize("x,rows,row_stride,head_stride,y,head_dim,code", [
    (0, 4, 768, 64, 0x2000, 64, -1),         # x NULL
    (0x1000, -1, 768, 64, 0x2000, 64, -1),   # negative row count
    (0x1000, 4, 768, 64, 0x2000, 60, -1),    # head_dim not a multiple of 8
    (0x1008, 4, 768, 64, 0x2000, 64, -3),    # x not 16-byte aligned
    (0x1000, 4, 768, 64, 0x2004, 64, -3),    # y not 8-byte aligned
    (0x1000, 4, 772, 64, 0x2000, 64, -3),    # row stride not a multiple of 8 elements
    (0x1000, 4, 768, 0, 0x2000, 64, -3),     # head stride not positive
])
def test_quantize_argument_errors(x, rows, row_stride, head_stride, y, head_dim, code):
    lib = _lib.load()
    rc = lib.fdb_quantize_e4m3(x or None, rows, row_stride, head_stride, 0x3000, 1, 12, head_dim, y, 0x4000, None)
    assert rc == code
    assert lib.fdb_last_error().decode() != ""


def test_quantize_zero_rows_is_a_no_op():
    lib = _lib.load()
    assert lib.fdb_quantize_e4m3(0x1000, 0, 768, 64, 0x3000, 1, 12, 64, 0x2000, 0x4000, None) == 0


@pytest.mark.parametrize("x,weight,k,n,code", [
    (0, 0x1000, 768, 3072, -1),        # x NULL
    (0x1000, 0, 768, 3072, -1),        # weight NULL
    (0x1000, 0x1000, 100, 3072, -2),   # in_features not a multiple of 64
    (0x1000, 0x1000, 768, 1000, -2),   # out_features not a multiple of 256
    (0x1008, 0x1000, 768, 3072, -3),   # x not 16-byte aligned
])
def test_linear_gelu_argument_errors(x, weight, k, n, code):
    lib = _lib.load()
    rc = lib.fdb_linear_gelu(x or None, weight or None, None, 0x2000, 4, k, n, None, None)
    assert rc == code
    assert lib.fdb_last_error().decode() != ""


def test_linear_gelu_zero_rows_is_a_no_op():
    lib = _lib.load()
    assert lib.fdb_linear_gelu(0x1000, 0x1000, None, 0x2000, 0, 768, 3072, None, None) == 0


@pytest.mark.parametrize("ids,table,rows_in_table,hidden,code", [
    (0, 0x1000, 100, 768, -1),         # ids NULL
    (0x1000, 0, 100, 768, -1),         # table NULL
    (0x1000, 0x1000, 0, 768, -1),      # empty table
    (0x1000, 0x1000, 100, 100, -2),    # hidden not a multiple of 256
    (0x1000, 0x1008, 100, 768, -3),    # table not 16-byte aligned
])
def test_embed_layernorm_argument_errors(ids, table, rows_in_table, hidden, code):
    lib = _lib.load()
    rc = lib.fdb_embed_layernorm(ids or None, table or None, rows_in_table, 0x1000, 0x1000, None, 0x2000, 4, hidden, 1e-7,
                                 None, None)
    assert rc == code
    assert lib.fdb_last_error().decode() != ""


def test_model_keeps_transformers_parameter_names():
    """Every block this package swaps in (embeddings, attention, intermediate and output blocks) keeps transformers'
    state-dict keys, so checkpoints load unchanged; on CPU tensors the blocks run transformers' own code."""
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    from flashdeberta_b200 import FlashDebertaV2Model
    cfg = DebertaV2Config(hidden_size=256, num_attention_heads=4, intermediate_size=512, num_hidden_layers=2,
                          relative_attention=True, position_buckets=32, max_relative_positions=64,
                          pos_att_type="c2p|p2c", share_att_key=True, vocab_size=100, type_vocab_size=0,
                          position_biased_input=False, norm_rel_ebd="layer_norm")
    cfg.attn_backend = "b200"
    ours, theirs = FlashDebertaV2Model(cfg).eval(), DebertaV2Model(cfg).eval()
    assert set(ours.state_dict().keys()) == set(theirs.state_dict().keys())
    theirs.load_state_dict(ours.state_dict())
    ids, mask = torch.randint(1, 100, (2, 9)), torch.ones(2, 9)
    with torch.no_grad():
        assert torch.equal(ours.embeddings(input_ids=ids, mask=mask), theirs.embeddings(input_ids=ids, mask=mask))
