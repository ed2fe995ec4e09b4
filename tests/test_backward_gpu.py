"""GPU parity tests of the attention backward: the two CUDA stages (csrc/attn_bwd.cu) behind
flashdeberta_b200.backward, the autograd wiring of the custom op, and training steps through the module and the model.

Reference gradients: autograd through the fp32 oracle on the host for the op-level tests (same bf16-grid inputs), the
eager backend of the same model with shared weights for the model-level tests.  The reference holds its own backward to
atol = rtol = 5e-3 in fp16 (tests/backward.py:99-102); here inputs, P and dS are bf16 (8 bits of mantissa), so a gradient
tensor is held to  max|got - want| <= 2e-2 * max|want|  and  mean|got - want| <= 2e-3 * max|want|.
"""
import pytest
import torch

from oracle import disentangled_attention as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_MAX, REL_MEAN = 2e-2, 2e-3


def _reference(q, k, v, pk, pq, starts, lens, sm, buckets, max_rel, dout):
    leaves = [t.float().cpu().clone().requires_grad_(True) if t is not None else None for t in (q, k, v, pk, pq)]
    with torch.enable_grad():
        out = oracle.attention_core.__wrapped__(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], starts, lens, sm,
                                                buckets, max_rel)
        grads = torch.autograd.grad(out, [t for t in leaves if t is not None], dout.float().cpu())
    it = iter(grads)
    return [next(it) if t is not None else None for t in leaves]


def _close(got, want, what, rel_max=REL_MAX, rel_mean=REL_MEAN):
    assert torch.isfinite(got.float()).all(), what
    scale = want.abs().max().item() + 1e-20
    diff = (got.float().cpu().reshape(want.shape) - want).abs()
    assert diff.max().item() <= rel_max * scale, (what, "max", diff.max().item() / scale)
    assert diff.mean().item() <= rel_mean * scale, (what, "mean", diff.mean().item() / scale)


def _run_op(q, k, v, pk, pq, dout, **kw):
    from flashdeberta_b200 import ops
    leaves = [t.clone().requires_grad_(True) if t is not None else None for t in (q, k, v, pk, pq)]
    out = ops.disentangled_attention(*leaves, **kw)
    assert out.requires_grad
    grads = torch.autograd.grad(out, [t for t in leaves if t is not None], dout)
    torch.cuda.synchronize()
    ops.check_status()
    it = iter(grads)
    return [next(it) if t is not None else None for t in leaves]


@pytest.mark.parametrize("buckets,max_rel,c2p,p2c", [(256, 512, True, True), (256, 512, True, False),
                                                     (256, 512, False, True), (-1, -1, False, False),
                                                     (-1, 128, True, True), (32, 64, True, True)])
def test_dense_ragged_gradients_vs_oracle_autograd(buckets, max_rel, c2p, p2c):
    g = torch.Generator().manual_seed(21)
    B, L, H, D = 2, 700, 2, 64
    lens = [700, 333]
    span = (buckets if buckets > 0 else max_rel) if (c2p or p2c) else 0
    q, k, v, dout = (torch.randn(B, L, H, D, generator=g).bfloat16().to(DEV) for _ in range(4))
    pk = torch.randn(H, 2 * span, D, generator=g).bfloat16().to(DEV) if c2p else None
    pq = torch.randn(H, 2 * span, D, generator=g).bfloat16().to(DEV) if p2c else None
    sm = oracle.sm_scale_for(D, c2p, p2c)
    got = _run_op(q, k, v, pk, pq, dout, seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV), max_seqlen=L,
                  sm_scale=sm, position_buckets=buckets, max_relative_positions=max_rel)
    flat = lambda t: t.reshape(-1, H, D)
    dmask = torch.zeros(B, L, 1, 1, device=DEV)
    for b, n in enumerate(lens):
        dmask[b, :n] = 1
    want = _reference(flat(q), flat(k), flat(v), pk, pq, [0, L], lens, sm, buckets, max_rel, flat(dout * dmask))
    for name, a, b in zip(("dq", "dk", "dv", "dpos_key", "dpos_query"), got, want):
        assert (a is None) == (b is None), name
        if a is not None:
            _close(a, b, name)
    assert got[0][1, 333:].abs().max().item() == 0 and got[2][1, 333:].abs().max().item() == 0


def test_packed_gradients_in_several_blocks_vs_oracle_autograd():
    """Packed sequences (an empty one, one of a single token, one of 1500) with the row blocks forced small, so that the p2c sums are
    accumulated over many blocks and the block edges fall inside the bucketed band."""
    from flashdeberta_b200 import backward, ops
    g = torch.Generator().manual_seed(22)
    H, D = 3, 64
    lens = [1500, 0, 1, 261]  # an empty sequence, a single token, an odd length
    cu = [0, 1500, 1500, 1501, 1762]
    T = cu[-1]
    q, k, v, dout = (torch.randn(T, H, D, generator=g).bfloat16().to(DEV) for _ in range(4))
    pk, pq = (torch.randn(H, 512, D, generator=g).bfloat16().to(DEV) for _ in range(2))
    sm = oracle.sm_scale_for(D, True, True)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=DEV)
    kw = dict(cu_seqlens=cu_t, max_seqlen=1500, sm_scale=sm, position_buckets=256, max_relative_positions=512)
    out, lse = ops.disentangled_attention(q, k, v, pk, pq, return_lse=True, **kw)
    got = backward.attention_backward(dout, q, k, v, pk, pq, out, lse, block_bytes=12 * H * 1500 * 192, **kw)
    whole = backward.attention_backward(dout, q, k, v, pk, pq, out, lse, **kw)
    torch.cuda.synchronize()
    want = _reference(q, k, v, pk, pq, cu[:-1], lens, sm, 256, 512, dout)
    for name, a, w, b in zip(("dq", "dk", "dv", "dpos_key", "dpos_query"), got, whole, want):
        _close(a, b, name)
        _close(w, b, name + " (one block)")


def test_gradients_at_2048_keys_with_far_tiles():
    """One sequence long enough that most keys of a row sit at the saturated ends of the tables (the long runs of the
    c2p sums) and that the forward inside the backward op takes its usual launches."""
    g = torch.Generator().manual_seed(23)
    L, H, D = 2048, 2, 64
    q, k, v, dout = (torch.randn(1, L, H, D, generator=g).bfloat16().to(DEV) for _ in range(4))
    pk, pq = (torch.randn(H, 512, D, generator=g).bfloat16().to(DEV) for _ in range(2))
    sm = oracle.sm_scale_for(D, True, True)
    got = _run_op(q, k, v, pk, pq, dout, max_seqlen=L, sm_scale=sm, position_buckets=256, max_relative_positions=512)
    want = _reference(q[0], k[0], v[0], pk, pq, [0], [L], sm, 256, 512, dout[0])
    for name, a, b in zip(("dq", "dk", "dv", "dpos_key", "dpos_query"), got, want):
        _close(a, b, name)


def _small_config(backend, **kw):
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    cfg = DebertaV2Config(vocab_size=2000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                          intermediate_size=512, relative_attention=True, position_buckets=256,
                          max_relative_positions=512, pos_att_type="c2p|p2c", share_att_key=True,
                          norm_rel_ebd="layer_norm", position_biased_input=False, type_vocab_size=0,
                          layer_norm_eps=1e-7, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                          pooler_dropout=0.0, cls_dropout=0.0, **kw)
    cfg.attn_backend = backend
    return cfg


@pytest.mark.parametrize("pack", [True, False])
def test_training_step_of_the_model_matches_the_eager_backend(pack):
    """loss.backward() through FlashDebertaV2ForSequenceClassification in train mode on a ragged batch: every parameter's
    gradient against the eager backend (fp32, same weights).  Packed and padded paths."""
    from flashdeberta_b200 import FlashDebertaV2ForSequenceClassification
    torch.manual_seed(3)
    ref = FlashDebertaV2ForSequenceClassification(_small_config("eager", num_labels=3)).to(DEV).float().train()
    cfg = _small_config("b200", num_labels=3)
    cfg.pack_sequences = pack
    fused = FlashDebertaV2ForSequenceClassification(cfg).to(DEV)
    fused.load_state_dict(ref.state_dict())
    fused = fused.bfloat16().train()
    g = torch.Generator().manual_seed(4)
    B, L, lens = 3, 400, (400, 222, 64)
    ids = torch.randint(1, 2000, (B, L), generator=g).to(DEV)
    mask = torch.zeros(B, L, device=DEV)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    labels = torch.tensor([0, 2, 1], device=DEV)
    loss_ref = ref(input_ids=ids, attention_mask=mask, labels=labels).loss
    loss_ref.backward()
    loss = fused(input_ids=ids, attention_mask=mask, labels=labels).loss
    loss.backward()
    torch.cuda.synchronize()
    assert abs(loss.item() - loss_ref.item()) < 5e-2
    checked = 0
    for (name, p_ref), (name2, p) in zip(ref.named_parameters(), fused.named_parameters()):
        assert name == name2
        if p_ref.grad is None:
            assert p.grad is None or p.grad.abs().max().item() == 0, name
            continue
        assert p.grad is not None, name
        scale = p_ref.grad.abs().max().item()
        if scale < 1e-6:
            continue
        diff = (p.grad.float() - p_ref.grad).abs()
        # whole bf16 model against an fp32 one: bf16 weights, activations and GEMMs on top of the attention itself
        assert diff.max().item() <= 0.15 * scale, (name, diff.max().item() / scale)
        assert diff.mean().item() <= 0.02 * scale, (name, diff.mean().item() / scale)
        checked += 1
    assert checked > 20
    attn = fused.deberta.encoder.layer[0].attention.self
    assert attn.query_proj.weight.grad.abs().max().item() > 0 and fused.deberta.encoder.rel_embeddings.weight.grad.abs().max().item() > 0


@pytest.mark.parametrize("varlen", [False, True])
def test_module_gradients_like_the_reference_suite(varlen):
    """The reference's backward test (tests/backward.py:66-200) on this module: 8 heads, 32 buckets / 64 positions, separate
    position projections, fixed-length and right-padded batches; gradients of the input, of the relative embeddings and
    of every parameter against transformers' module in fp32 (the reference compares in fp16 with atol = rtol = 5e-3; the
    bf16 module is held to 3e-2 of each gradient's largest entry)."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention
    from flashdeberta_b200 import FlashDisentangledSelfAttention

    class Cfg:
        hidden_size, num_attention_heads = 512, 8
        attention_probs_dropout_prob = hidden_dropout_prob = 0.0
        pos_att_type, relative_attention = ["c2p", "p2c"], True
        position_buckets, max_relative_positions, max_position_embeddings, share_att_key = 32, 64, 512, False

    torch.manual_seed(0)
    eager = DisentangledSelfAttention(Cfg()).to(DEV).eval()
    with torch.no_grad():
        for p in eager.parameters():
            p.copy_(p.bfloat16().float())
    flash = FlashDisentangledSelfAttention(Cfg()).to(DEV).eval()
    flash.load_state_dict(eager.state_dict())
    flash = flash.bfloat16()
    g = torch.Generator().manual_seed(1)
    B, L = 3, 384
    hs = torch.randn(B, L, 512, generator=g).bfloat16().float().to(DEV)
    rel = torch.randn(64, 512, generator=g).bfloat16().float().to(DEV)
    mask = torch.ones(B, L, device=DEV)
    if varlen:
        for b, n in enumerate((384, 201, 17)):
            mask[b, n:] = 0
    ext = mask.unsqueeze(1).unsqueeze(2)
    ext = ext * ext.squeeze(-2).unsqueeze(-1)
    grad_out = torch.randn(B, L, 512, generator=g).to(DEV) * mask.unsqueeze(-1)

    hs_a, rel_a = hs.clone().requires_grad_(True), rel.clone().requires_grad_(True)
    (eager(hs_a, ext, rel_embeddings=rel_a)[0] * grad_out).sum().backward()
    hs_b, rel_b = hs.bfloat16().requires_grad_(True), rel.bfloat16().requires_grad_(True)
    (flash(hs_b, mask, rel_embeddings=rel_b)[0].float() * grad_out).sum().backward()
    torch.cuda.synchronize()

    def check(name, got, want):
        scale = want.abs().max().item()
        diff = (got.float() - want).abs().max().item()
        # the reference's own criterion has the same absolute floor (tests/backward.py:52-54): pos_key_proj.bias shifts
        # every score of a row alike, its true gradient is zero and what is compared there is rounding noise
        assert diff <= 3e-2 * scale or diff <= 5e-3, (name, diff, scale)

    check("hidden_states", hs_b.grad, hs_a.grad)
    check("rel_embeddings", rel_b.grad, rel_a.grad)
    n_checked = 0
    for (name, pa), (_, pb) in zip(eager.named_parameters(), flash.named_parameters()):
        if pa.grad is None:
            continue
        assert pb.grad is not None, name
        check(name, pb.grad, pa.grad)
        n_checked += 1
    assert n_checked >= 8  # q, k, v and the two position projections, weights and biases


def test_backward_through_the_compiled_module():
    """The attention module traced as one graph (forward op and backward op both opaque nodes) gives the eager-mode
    gradients of the same module."""
    from flashdeberta_b200 import FlashDisentangledSelfAttention
    cfg = _small_config("b200")
    torch.manual_seed(5)
    mod = FlashDisentangledSelfAttention(cfg).to(DEV).bfloat16().train()
    g = torch.Generator().manual_seed(6)
    x = torch.randn(2, 256, 256, generator=g).bfloat16().to(DEV)
    rel = torch.randn(512, 256, generator=g).bfloat16().to(DEV)
    mask = torch.ones(2, 256, device=DEV)
    mask[1, 200:] = 0

    def grads(fn):
        xs = x.clone().requires_grad_(True)
        mod.zero_grad()
        out = fn(xs, mask, rel_embeddings=rel)[0]
        out.float().square().sum().backward()
        return xs.grad.clone(), mod.query_proj.weight.grad.clone()

    eager = grads(mod)
    compiled = grads(torch.compile(mod, fullgraph=True, backend="aot_eager"))
    for a, b in zip(eager, compiled):  # same kernels; the p2c sums add in shared memory in no fixed order
        assert (a.float() - b.float()).abs().max().item() <= 1e-2 * b.float().abs().max().item()


def test_fp8_attention_refuses_to_train():
    from flashdeberta_b200 import ops
    q = torch.randn(1, 128, 2, 64, device=DEV).bfloat16().requires_grad_(True)
    with pytest.raises(RuntimeError, match="forward-only"):
        ops.disentangled_attention_fp8(q, q, q, None, None, max_seqlen=128)
