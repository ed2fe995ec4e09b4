"""GPU parity tests on the benchmark configurations themselves and on the parts of the Python surface the other files do
not reach: the packed 256-sequence batch (16 heads), the e4m3 layer shape (4096 keys, 16 heads) and a 24-layer e4m3
encoder, ``query_states``, the torch custom op (direct, traced, opcheck), every task head, save/load, mask layouts,
``torch.inference_mode``, ``z_steps`` and the packed-ids model entry.

Tolerances: bf16 fused attention vs the fp32 oracle max-abs <= 2e-2, mean-abs <= 2e-3.  FP8 single layer vs fp32:
max-abs <= 2e-2, mean-abs <= 3e-3 at DeBERTa magnitudes (weights N(0, 0.02)).  Whole encoders are compared on their
LayerNorm outputs (|x| ~ 1): bf16 encoder vs fp32 eager max-abs <= 0.25, mean-abs <= 0.02; FP8 attention inside a 24-layer
encoder is held to max-abs <= 0.25, mean-abs <= 0.025 (first measurement on a B200: 0.088 / 0.0122, with bf16 attention
0.090 / 0.0117 on the same weights and ids).
"""
import math

import pytest
import torch

from oracle import disentangled_attention as oracle

pytestmark = pytest.mark.gpu

BF16_MAX, BF16_MEAN = 2e-2, 2e-3
ENC_MAX, ENC_MEAN = 0.25, 0.02
FP8_ENC_MAX, FP8_ENC_MEAN = 0.25, 0.025
DEV = "cuda"


def _ops():
    from flashdeberta_b200 import ops
    return ops


def _close(got, want, max_tol, mean_tol, what=""):
    diff = (got.float().cpu() - want.float().cpu()).abs()
    assert torch.isfinite(got.float()).all(), what
    assert diff.max().item() <= max_tol, (what, "max-abs", diff.max().item())
    assert diff.mean().item() <= mean_tol, (what, "mean-abs", diff.mean().item())


def packed_batch_lengths():
    """The 256 sequence lengths of the packed benchmark batch: log-uniform in [64, 8192] from seed 2."""
    g = torch.Generator(device="cpu").manual_seed(2)
    u = torch.rand(256, dtype=torch.float64, generator=g)
    return torch.floor(torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))).long().tolist()


# ---------------------------------------------------------------------------------------------------------------------
# the packed 256-sequence batch, 16 heads: one call, the library chooses its launches
# ---------------------------------------------------------------------------------------------------------------------
def test_packed_256_sequence_batch_vs_oracle_and_alone():
    ops = _ops()
    lens = packed_batch_lengths()
    assert sum(lens) == 350907 and lens[:8] == [5491, 102, 1993, 880, 5377, 820, 114, 233]
    assert min(lens) == 65 and max(lens) == 7995
    T, H, D = sum(lens), 16, 64
    g = torch.Generator(device=DEV).manual_seed(2)
    q, k, v = (torch.randn(T, H, D, generator=g, device=DEV, dtype=torch.float32).bfloat16() for _ in range(3))
    pk, pq = (torch.randn(H, 512, D, generator=g, device=DEV, dtype=torch.float32).bfloat16() for _ in range(2))
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    kw = dict(position_buckets=256, max_relative_positions=512)
    out = ops.disentangled_attention(q, k, v, pk, pq, cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=DEV),
                                     max_seqlen=max(lens), **kw)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.isfinite(out.float()).all()

    order = sorted(range(256), key=lambda i: lens[i])
    mid = [i for i in order if 3584 <= lens[i] <= 8192]
    near128 = sorted(range(256), key=lambda i: min(lens[i] % 128, 128 - lens[i] % 128))
    picks = [order[0], order[-1], mid[0], mid[len(mid) // 2], near128[0], near128[1], order[128], order[200]]
    sm = oracle.sm_scale_for(D, True, True)
    for n_pick, b in enumerate(dict.fromkeys(picks)):
        s0, n = cu[b], lens[b]
        h = (5 * n_pick + 3) % H
        sl = slice(s0, s0 + n)
        # the same sequence alone (dense, one sequence): bit-identical, whatever the batch around it
        alone = ops.disentangled_attention(q[sl].unsqueeze(0), k[sl].unsqueeze(0), v[sl].unsqueeze(0), pk, pq,
                                           max_seqlen=n, **kw)
        assert torch.equal(alone[0], out[sl]), (b, n)
        want = oracle.attention_core(q[sl, h:h + 1].float().cpu(), k[sl, h:h + 1].float().cpu(),
                                     v[sl, h:h + 1].float().cpu(), pk[h:h + 1].float().cpu(), pq[h:h + 1].float().cpu(),
                                     [0], [n], sm, 256, 512)
        _close(out[sl, h:h + 1], want, BF16_MAX, BF16_MEAN, f"sequence {b} (length {n}) head {h}")
    ops.check_status()


# ---------------------------------------------------------------------------------------------------------------------
# e4m3 at the layer shape of the FP8 configuration: 4096 keys, 16 heads
# ---------------------------------------------------------------------------------------------------------------------
def test_fp8_layer_shape_4096_keys_16_heads():
    ops = _ops()
    B, L, H, D = 2, 4096, 16, 64
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(B, L, H, D, generator=g).bfloat16() for _ in range(3))
    pk, pq = (torch.randn(H, 512, D, generator=g).bfloat16() for _ in range(2))
    sm = oracle.sm_scale_for(D, True, True)
    out = ops.disentangled_attention_fp8(q.to(DEV), k.to(DEV), v.to(DEV), pk.to(DEV), pq.to(DEV), max_seqlen=L, sm_scale=sm,
                                         position_buckets=256, max_relative_positions=512)
    torch.cuda.synchronize()
    ops.check_status()
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    fq = lambda x: oracle.fake_quant_e4m3(x.float(), dims=(1, 3))[0].bfloat16()   # per (sequence, head)
    ft = lambda x: oracle.fake_quant_e4m3(x.float(), dims=(1, 2))[0].bfloat16()   # per head
    qq, kq, vq, pkq, pqq = fq(q), fq(k), fq(v), ft(pk), ft(pq)
    for b, h in [(0, 0), (1, 15), (0, 9)]:
        one = lambda t: t[b, :, h:h + 1].float()
        want = oracle.attention_core(one(q), one(k), one(v), pk[h:h + 1].float(), pq[h:h + 1].float(), [0], [L], sm, 256, 512)
        expect = oracle.attention_core(one(qq), one(kq), one(vq), pkq[h:h + 1].float(), pqq[h:h + 1].float(), [0], [L], sm,
                                       256, 512)
        d_exp = (got[b, :, h:h + 1] - expect).abs()   # what is left is the e4m3 rounding of P
        assert d_exp.max().item() <= 3e-2 and d_exp.mean().item() <= 4e-3, (b, h, d_exp.max().item(), d_exp.mean().item())
        d_q = (expect - want).abs()
        d = (got[b, :, h:h + 1] - want).abs()
        assert d.max().item() <= 1.5 * d_q.max().item() + 3e-2 and d.mean().item() <= 1.5 * d_q.mean().item() + 4e-3


def _large_config(layers=24, backend="b200", fp8=False):
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    cfg = DebertaV2Config(
        vocab_size=128100, hidden_size=1024, num_hidden_layers=layers, num_attention_heads=16, intermediate_size=4096,
        hidden_act="gelu", max_position_embeddings=512, type_vocab_size=0, layer_norm_eps=1e-7, relative_attention=True,
        max_relative_positions=-1, position_buckets=256, norm_rel_ebd="layer_norm", share_att_key=True,
        pos_att_type="c2p|p2c", position_biased_input=False, pad_token_id=0, hidden_dropout_prob=0.0,
        attention_probs_dropout_prob=0.0)
    cfg.attn_backend, cfg.attn_fp8 = backend, fp8
    return cfg


def test_fp8_24_layer_encoder_vs_fp32_eager():
    """DeBERTa-v3-large shape, random-init (seed 4), 1 x 1024 tokens: e4m3 attention inside the bf16 encoder against the
    fp32 eager encoder, with the bf16 attention beside it."""
    from flashdeberta_b200 import FlashDebertaV2Model
    torch.manual_seed(4)
    eager = FlashDebertaV2Model(_large_config(backend="eager")).eval().to(DEV)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(1, 128100, (1, 1024), generator=g).to(DEV)
    mask = torch.ones(1, 1024, device=DEV)
    with torch.no_grad():
        want = eager(input_ids=ids, attention_mask=mask).last_hidden_state
        res = {}
        for name, fp8 in (("bf16", False), ("fp8", True)):
            m = FlashDebertaV2Model(_large_config(fp8=fp8)).eval()
            m.load_state_dict(eager.state_dict())
            m = m.to(DEV).bfloat16()
            got = m(input_ids=ids, attention_mask=mask).last_hidden_state
            d = (got.float() - want).abs()
            res[name] = (d.max().item(), d.mean().item())
            del m
    _ops().check_status()
    print("24-layer encoder vs fp32 eager (max-abs, mean-abs):", res)
    assert res["bf16"][0] <= ENC_MAX and res["bf16"][1] <= ENC_MEAN, res
    assert res["fp8"][0] <= FP8_ENC_MAX and res["fp8"][1] <= FP8_ENC_MEAN, res


# ---------------------------------------------------------------------------------------------------------------------
# module surface: query_states, the custom op
# ---------------------------------------------------------------------------------------------------------------------
class _Cfg:
    def __init__(self, hidden, heads, buckets=256, max_rel=512, pat=("c2p", "p2c"), share=True):
        self.hidden_size, self.num_attention_heads = hidden, heads
        self.attention_probs_dropout_prob = self.hidden_dropout_prob = 0.1
        self.pos_att_type, self.relative_attention = list(pat), True
        self.position_buckets, self.max_relative_positions = buckets, max_rel
        self.max_position_embeddings, self.share_att_key = 512, share


def _module_pair(hidden, heads, seed=0, **kw):
    from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention
    from flashdeberta_b200 import FlashDisentangledSelfAttention
    g = torch.Generator().manual_seed(seed)
    cfg = _Cfg(hidden, heads, **kw)
    eager = DisentangledSelfAttention(cfg).eval()
    with torch.no_grad():
        for p in eager.parameters():
            p.copy_((torch.randn(p.shape, generator=g) * 0.02).bfloat16().float())
    flash = FlashDisentangledSelfAttention(cfg).eval()
    flash.load_state_dict(eager.state_dict())
    return eager.to(DEV), flash.to(DEV).bfloat16(), g


def _ext(mask):
    e = mask.unsqueeze(1).unsqueeze(2)
    return e * e.squeeze(-2).unsqueeze(-1)


def test_module_query_states_vs_live_eager():
    """Queries projected from another tensor than keys and values (src/flashdeberta/model.py:132-133)."""
    eager, flash, g = _module_pair(256, 4, share=False)
    B, L = 2, 700
    hs = torch.randn(B, L, 256, generator=g).bfloat16().float().to(DEV)
    qs = torch.randn(B, L, 256, generator=g).bfloat16().float().to(DEV)
    rel = (torch.randn(512, 256, generator=g) * 0.02).bfloat16().float().to(DEV)
    mask = torch.ones(B, L, device=DEV)
    mask[1, 450:] = 0
    with torch.no_grad():
        want = eager(hs, _ext(mask), query_states=qs, rel_embeddings=rel)[0]
        got = flash(hs.bfloat16(), mask, query_states=qs.bfloat16(), rel_embeddings=rel.bfloat16())[0]
        plain = flash(hs.bfloat16(), mask, rel_embeddings=rel.bfloat16())[0]
    valid = mask.bool().unsqueeze(-1)
    _close(got * valid, want * valid, BF16_MAX, BF16_MEAN, "query_states")
    assert not torch.equal(got, plain)
    _ops().check_status()


def test_module_head_size_128_runs_on_the_general_kernel():
    """Head size 128 (the one such shape in the reference's test, tests/attention.py:87-89): the module takes the library's
    general kernel, dense and packed; training there is refused."""
    import warnings
    from flashdeberta_b200.attention import PackedSequences
    eager, flash, g = _module_pair(256, 2)  # 256 / 2 heads = 128
    B, L = 2, 260
    hs = torch.randn(B, L, 256, generator=g).bfloat16().float().to(DEV)
    rel = (torch.randn(512, 256, generator=g) * 0.02).bfloat16().float().to(DEV)
    mask = torch.ones(B, L, device=DEV)
    mask[1, 99:] = 0
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = eager(hs, _ext(mask), rel_embeddings=rel)[0]
        got = flash(hs.bfloat16(), mask, rel_embeddings=rel.bfloat16())[0]
        packed = PackedSequences.from_mask(mask)
        got_p = packed.unpack(flash(packed.pack(hs.bfloat16()), packed, rel_embeddings=rel.bfloat16())[0])
    valid = mask.bool().unsqueeze(-1)
    _close(got * valid, want * valid, BF16_MAX, BF16_MEAN, "head size 128, dense")
    _close(got_p * valid, want * valid, BF16_MAX, BF16_MEAN, "head size 128, packed")
    assert got[1, 99:].abs().max().item() == 0
    with pytest.raises(RuntimeError, match="head size of 64"), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        flash.train()(hs.bfloat16().requires_grad_(True), mask, rel_embeddings=rel.bfloat16())
    _ops().check_status()


def test_reference_suite_shape_in_fp32():
    """The one case of the reference's own forward test (tests/attention.py:81-104): batch 1 x 2048 tokens, hidden 1024,
    8 heads (head size 128), fp32 modules, all-ones mask, separate position projections; its bar is a mean absolute
    difference below 1e-4 against transformers' module."""
    import warnings
    eager, flash, g = _module_pair(1024, 8, share=False)
    flash = flash.float()
    hs = torch.randn(1, 2048, 1024, generator=g).to(DEV)
    rel = torch.randn(512, 1024, generator=g).to(DEV)
    mask = torch.ones(1, 2048, device=DEV)
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        want = eager(hs, _ext(mask), rel_embeddings=rel)[0]
        got = flash(hs, mask, rel_embeddings=rel)[0]
    assert got.dtype == torch.float32
    diff = (got - want).abs()
    assert diff.mean().item() < 1e-4, diff.mean().item()
    assert diff.max().item() < 1e-3, diff.max().item()
    _ops().check_status()


def test_custom_op_direct_traced_and_opcheck():
    """flashdeberta_b200::attn_fwd, the torch-facing boundary: called directly, through the module under torch.compile
    (whole graph, fake tensors propagated through register_fake) and through torch.library.opcheck."""
    ops = _ops()
    eager, flash, g = _module_pair(256, 4)
    B, L, H, D = 2, 300, 4, 64
    q, k, v = (torch.randn(B, L, H, D, generator=g).bfloat16().to(DEV) for _ in range(3))
    pk, pq = (torch.randn(H, 512, D, generator=g).bfloat16().to(DEV) for _ in range(2))
    lens = torch.tensor([300, 170], dtype=torch.int32, device=DEV)
    sm = oracle.sm_scale_for(D, True, True)
    want = ops.disentangled_attention(q, k, v, pk, pq, seq_lens=lens, max_seqlen=L, sm_scale=sm, position_buckets=256,
                                      max_relative_positions=512)
    got = torch.ops.flashdeberta_b200.attn_fwd(q, k, v, pk, pq, None, lens, L, sm, 256, 512)
    assert torch.equal(got, want)
    # packed form and absent tables through the op schema
    cu = torch.tensor([0, 300, 470], dtype=torch.int32, device=DEV)
    qp = torch.cat([q[0], q[1, :170]]); kp = torch.cat([k[0], k[1, :170]]); vp = torch.cat([v[0], v[1, :170]])
    got_p = torch.ops.flashdeberta_b200.attn_fwd(qp, kp, vp, pk, pq, cu, None, L, sm, 256, 512)
    assert torch.equal(got_p[:300], want[0]) and torch.equal(got_p[300:], want[1, :170])
    torch.ops.flashdeberta_b200.attn_fwd(q, k, v, None, None, None, None, L, 0.125, -1, -1)
    # fake-tensor propagation: shape and dtype without running anything
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode() as mode:
        fq = mode.from_tensor(q)
        fo = torch.ops.flashdeberta_b200.attn_fwd(fq, fq, fq, None, None, None, None, L, 0.125, -1, -1)
        assert fo.shape == q.shape and fo.dtype == torch.bfloat16
    torch.library.opcheck(torch.ops.flashdeberta_b200.attn_fwd.default, (q, k, v, pk, pq, None, lens, L, sm, 256, 512),
                          test_utils=("test_schema", "test_faketensor"))
    # the op records a backward (tests/test_backward_gpu.py holds it to the oracle's autograd); opcheck on its registration
    qg = q.clone().requires_grad_(True)
    o = torch.ops.flashdeberta_b200.attn_fwd(qg, k, v, pk, pq, None, lens, L, sm, 256, 512)
    o.float().sum().backward()
    assert qg.grad is not None and torch.isfinite(qg.grad.float()).all() and qg.grad[1, 170:].abs().max().item() == 0
    torch.library.opcheck(torch.ops.flashdeberta_b200.attn_fwd.default, (qg.detach().requires_grad_(True), k, v, pk, pq, None, lens, L, sm, 256, 512),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    # the module traced as one graph: the attention is the custom-op node
    hs = torch.randn(B, L, 256, generator=g).bfloat16().to(DEV)
    rel = (torch.randn(512, 256, generator=g) * 0.02).bfloat16().to(DEV)
    mask = torch.ones(B, L, device=DEV)
    mask[1, 170:] = 0
    with torch.no_grad():
        ref = flash(hs, mask, rel_embeddings=rel)[0]
        compiled = torch.compile(flash, fullgraph=True, backend="aot_eager")
        out = compiled(hs, mask, rel_embeddings=rel)[0]
    _close(out, ref, 1e-6, 1e-7, "traced module")
    torch.cuda.synchronize()
    ops.check_status()


# ---------------------------------------------------------------------------------------------------------------------
# model level: the five heads, save / load, masks, inference mode, z_steps, packed ids
# ---------------------------------------------------------------------------------------------------------------------
def _small_config(backend, **kw):
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    cfg = DebertaV2Config(vocab_size=2000, hidden_size=256, num_hidden_layers=3, num_attention_heads=4,
                          intermediate_size=512, relative_attention=True, position_buckets=256,
                          max_relative_positions=512, pos_att_type="c2p|p2c", share_att_key=True,
                          norm_rel_ebd="layer_norm", position_biased_input=False, type_vocab_size=0,
                          layer_norm_eps=1e-7, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                          pooler_dropout=0.0, cls_dropout=0.0, **kw)
    cfg.attn_backend = backend
    return cfg


def _ragged(B=3, L=500, lens=(500, 333, 90), vocab=2000, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(1, vocab, (B, L), generator=g).to(DEV)
    mask = torch.zeros(B, L, device=DEV)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    return ids, mask


@pytest.mark.parametrize("head", ["MaskedLM", "SequenceClassification", "TokenClassification", "QuestionAnswering",
                                  "MultipleChoice"])
def test_task_heads_vs_eager_backend(head):
    """Each exported head (src/flashdeberta/model.py:498-920) on the fused backend against the same head, same weights, on
    transformers' eager attention in fp32."""
    import flashdeberta_b200 as pkg
    cls = getattr(pkg, "FlashDebertaV2For" + head)
    torch.manual_seed(0)
    labels = 2 if head == "QuestionAnswering" else 3
    eager = cls(_small_config("eager", num_labels=labels)).eval().to(DEV)
    fused = cls(_small_config("b200", num_labels=labels)).eval()
    fused.load_state_dict(eager.state_dict())
    fused = fused.to(DEV).bfloat16()
    ids, mask = _ragged()
    if head == "MultipleChoice":  # (batch, choices, L): the head flattens to (batch * choices, L) and back
        ids2, mask2 = _ragged(seed=1)
        ids, mask = torch.stack([ids, ids2], 1), torch.stack([mask, mask2], 1)
    with torch.no_grad():
        want = eager(input_ids=ids, attention_mask=mask)
        got = fused(input_ids=ids, attention_mask=mask)
    names = ["start_logits", "end_logits"] if head == "QuestionAnswering" else ["logits"]
    for n in names:
        w, o = getattr(want, n), getattr(got, n)
        assert o.shape == w.shape
        if head in ("MaskedLM", "TokenClassification"):  # per-token outputs: valid tokens only
            valid = mask.bool().unsqueeze(-1)
            w, o = w * valid, o.float() * valid
        if head == "QuestionAnswering":
            w, o = w * mask, o.float() * mask
        # logits are a linear read-out of the encoder output: held to the whole-encoder bound
        _close(o, w, ENC_MAX, ENC_MEAN, f"{head}.{n}")
    if head == "MultipleChoice":
        assert got.logits.shape == (3, 2)
    _ops().check_status()


def test_save_pretrained_from_pretrained_round_trip(tmp_path):
    from flashdeberta_b200 import FlashDebertaV2Model
    torch.manual_seed(0)
    model = FlashDebertaV2Model(_small_config("b200")).eval().to(DEV).bfloat16()
    ids, mask = _ragged()
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).last_hidden_state
    model.save_pretrained(tmp_path)
    again = FlashDebertaV2Model.from_pretrained(tmp_path).eval().to(DEV).bfloat16()
    assert getattr(again.config, "attn_backend", "b200") == "b200" and again.encoder._fused
    with torch.no_grad():
        got = again(input_ids=ids, attention_mask=mask).last_hidden_state
    assert torch.equal(got, want)
    # a stock transformers checkpoint (same parameter names) loads too
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    stock = DebertaV2Model(_small_config("b200")).eval()
    stock.load_state_dict({k: v.float().cpu() for k, v in model.state_dict().items()})
    stock.save_pretrained(tmp_path / "stock")
    third = FlashDebertaV2Model.from_pretrained(tmp_path / "stock").eval().to(DEV).bfloat16()
    with torch.no_grad():
        assert torch.equal(third(input_ids=ids, attention_mask=mask).last_hidden_state, want)


def test_mask_layouts():
    """A dense mask is addressed by length alone, so it must be right-padded: a mask on the host that is not raises; one
    on the device sets FDB_DEV_BAD_MASK.  The model packs padded batches and so takes any layout; a left-padded batch gives
    what the eager backend gives."""
    from flashdeberta_b200 import FlashDebertaV2Model, ops
    from flashdeberta_b200.attention import lengths_from_mask
    right = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]])
    left = torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]])
    holes = torch.tensor([[1, 0, 1, 1, 0], [1, 1, 1, 1, 1]])
    assert lengths_from_mask(right).tolist() == [3, 5]
    assert lengths_from_mask(_ext(right.float())).tolist() == [3, 5]
    for bad in (left, holes, _ext(left.float())):
        with pytest.raises(ValueError, match="right-padded"):
            lengths_from_mask(bad)
    assert lengths_from_mask(right.to(DEV)).tolist() == [3, 5]
    ops.check_status()
    for bad in (left, _ext(holes.float())):
        lengths_from_mask(bad.to(DEV))
        with pytest.raises(RuntimeError, match="right-padded"):
            ops.check_status()
    ops.check_status()  # cleared

    torch.manual_seed(0)
    eager = FlashDebertaV2Model(_small_config("eager")).eval().to(DEV)
    fused = FlashDebertaV2Model(_small_config("b200")).eval()
    fused.load_state_dict(eager.state_dict())
    fused = fused.to(DEV).bfloat16()
    B, L = 3, 400
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(1, 2000, (B, L), generator=g).to(DEV)
    mask = torch.zeros(B, L, device=DEV)
    mask[0, :] = 1
    mask[1, 150:] = 1   # left-padded
    mask[2, 390:] = 1
    with torch.no_grad():
        want = eager(input_ids=ids, attention_mask=mask).last_hidden_state
        got = fused(input_ids=ids, attention_mask=mask).last_hidden_state
    valid = mask.bool().unsqueeze(-1)
    _close(got.float() * valid, want * valid, ENC_MAX, ENC_MEAN, "left-padded batch")
    assert torch.count_nonzero(got * ~valid) == 0
    ops.check_status()
    # with packing off the same batch is refused through the status word instead of being computed wrongly
    cfg = _small_config("b200")
    cfg.pack_sequences = False
    padded = FlashDebertaV2Model(cfg).eval()
    padded.load_state_dict(eager.state_dict())
    padded = padded.to(DEV).bfloat16()
    with torch.no_grad():
        padded(input_ids=ids, attention_mask=mask)
    with pytest.raises(RuntimeError, match="right-padded"):
        ops.check_status()


def test_inference_mode():
    """Tensors made under torch.inference_mode keep no version counter; the caches that key on one must cope."""
    from flashdeberta_b200 import FlashDebertaV2Model, ops
    torch.manual_seed(0)
    model = FlashDebertaV2Model(_small_config("b200")).eval().to(DEV).bfloat16()
    ids, mask = _ragged()
    full = torch.ones_like(mask)
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).last_hidden_state
        want_full = model(input_ids=ids, attention_mask=full).last_hidden_state
    fresh = FlashDebertaV2Model(_small_config("b200")).eval()
    fresh.load_state_dict(model.state_dict())
    fresh = fresh.to(DEV).bfloat16()
    with torch.inference_mode():
        for _ in range(2):  # the second pass meets what the first one cached
            assert torch.equal(fresh(input_ids=ids, attention_mask=mask).last_hidden_state, want)
            assert torch.equal(fresh(input_ids=ids, attention_mask=torch.ones_like(mask)).last_hidden_state, want_full)
        # the op layer with a workspace kept between calls
        g = torch.Generator().manual_seed(1)
        q, k, v = (torch.randn(2, 200, 4, 64, generator=g).bfloat16().to(DEV) for _ in range(3))
        pk, pq = (torch.randn(4, 512, 64, generator=g).bfloat16().to(DEV) for _ in range(2))
        lens = torch.tensor([200, 77], dtype=torch.int32, device=DEV)
        prepared = ops.PreparedWorkspace()
        kw = dict(seq_lens=lens, max_seqlen=200, position_buckets=256, max_relative_positions=512)
        a = ops.disentangled_attention(q, k, v, pk, pq, prepared=prepared, **kw)
        b = ops.disentangled_attention(q, k, v, pk, pq, prepared=prepared, **kw)
        c = ops.disentangled_attention(q, k, v, pk, pq, **kw)
        assert torch.equal(a, c) and torch.equal(b, c)
    ops.check_status()


def test_z_steps_repeats_the_last_layer():
    """z_steps = 2: the last layer once more, queries = its previous output, keys and values = the output of the layer
    before (the intent of src/flashdeberta/model.py:469-485), against the same steps on the eager backend in fp32."""
    from flashdeberta_b200 import FlashDebertaV2Model
    torch.manual_seed(0)
    eager = FlashDebertaV2Model(_small_config("eager")).eval().to(DEV)
    fused = FlashDebertaV2Model(_small_config("b200")).eval()
    fused.load_state_dict(eager.state_dict())
    fused = fused.to(DEV).bfloat16()
    fused.z_steps = 2
    ids, mask = _ragged()
    with torch.no_grad():
        base = eager(input_ids=ids, attention_mask=mask, output_hidden_states=True)
        enc = eager.encoder
        want = enc.layer[-1](base.hidden_states[-2], enc.get_attention_mask(mask), query_states=base.hidden_states[-1],
                             relative_pos=enc.get_rel_pos(base.hidden_states[0]), rel_embeddings=enc.get_rel_embedding())[0]
        got = fused(input_ids=ids, attention_mask=mask, output_hidden_states=True)
    assert len(got.hidden_states) == len(base.hidden_states) + 1
    valid = mask.bool().unsqueeze(-1)
    _close(got.last_hidden_state.float() * valid, want * valid, ENC_MAX, ENC_MEAN, "z_steps")
    assert not torch.equal(got.last_hidden_state, got.hidden_states[-2])
    _ops().check_status()


def test_model_packed_ids_entry():
    """Packed ids + cu_seqlens straight into the model: the same bits as the padded batch it stands for."""
    from flashdeberta_b200 import FlashDebertaV2Model
    torch.manual_seed(0)
    model = FlashDebertaV2Model(_small_config("b200")).eval().to(DEV).bfloat16()
    lens = (500, 333, 90)
    ids, mask = _ragged(lens=lens)
    packed_ids = torch.cat([ids[b, :n] for b, n in enumerate(lens)])
    cu = torch.tensor([0, 500, 833, 923], dtype=torch.int32, device=DEV)
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).last_hidden_state
        got = model(input_ids=packed_ids, cu_seqlens=cu, max_seqlen=500).last_hidden_state
    assert got.shape == (1, 923, 256)
    at = 0
    for b, n in enumerate(lens):
        assert torch.equal(got[0, at:at + n], want[b, :n]), b
        at += n
    _ops().check_status()
