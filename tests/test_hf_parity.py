"""The oracle decoder against Hugging Face's GPT-2: same state-dict keys and tensor layout (Conv1D
``[in, out]`` weights, tied lm_head), and the same logits from the same weights.  This is what makes
checkpoints interchangeable with the reference, whose model is ``GPT2LMHeadModel`` inside the two
wrappers (``src/modeling/model.py:19-20,69-70,165-179``)."""
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _models():
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    ours = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                            n_embd=64, n_head=2, n_positions=64, resid_pdrop=0.0, embd_pdrop=0.0,
                            attn_pdrop=0.0)
    cfg = transformers.GPT2Config(vocab_size=len(tok), n_positions=64, n_embd=64, n_layer=2, n_head=2,
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                                  activation_function="gelu_new")
    hf = transformers.GPT2LMHeadModel(cfg)
    return tok, ours.eval(), hf.eval()


def test_state_dict_keys_and_shapes_match_hf_gpt2():
    tok, ours, hf = _models()
    inner = {k[len("model.model."):]: v for k, v in ours.state_dict().items() if k.startswith("model.model.")}
    want = {k: v for k, v in hf.state_dict().items() if not k.endswith(".attn.bias") and not k.endswith(".attn.masked_bias")}
    assert set(inner) == set(want), (sorted(set(inner) ^ set(want)))
    for k, v in want.items():
        assert tuple(inner[k].shape) == tuple(v.shape), k
    # what the wrappers add on top of the HF module
    extra = sorted(k for k in ours.state_dict() if not k.startswith("model.model."))
    assert extra == ["model.control_embeds.weight", "time_head.0.bias", "time_head.0.weight",
                     "value_head.0.bias", "value_head.0.weight"]


def test_logits_match_hf_gpt2_on_the_same_weights():
    tok, ours, hf = _models()
    sd = {k: v for k, v in hf.state_dict().items() if not k.endswith(".attn.bias") and not k.endswith(".attn.masked_bias")}
    inner = ours.model.model
    missing, unexpected = inner.load_state_dict(sd, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    ids = torch.randint(0, 1968, (3, 40))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = inner(input_ids=ids)
    got = got["logits"] if isinstance(got, dict) else (got.logits if hasattr(got, "logits") else got)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max().item()


def test_use_pretrained_loads_a_local_gpt2_body(tmp_path):
    """``use_pretrained`` with ``base_model`` = a local HF directory: every block weight and the
    position table come from the checkpoint, the token embedding is re-drawn with the pretrained
    embedding's mean and spread (its vocabulary is text, not chess moves)."""
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model

    torch.manual_seed(1)
    cfg = transformers.GPT2Config(vocab_size=500, n_positions=64, n_embd=64, n_layer=2, n_head=2,
                                  activation_function="gelu_new")
    hf = transformers.GPT2LMHeadModel(cfg)
    with torch.no_grad():
        hf.transformer.wte.weight.mul_(5.0).add_(0.3)
    hf.save_pretrained(tmp_path / "gpt2-local")
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    ours = initialize_model(tok, str(tmp_path / "gpt2-local"), use_control_token=True, use_regression_head=True,
                            use_pretrained=True)
    inner = ours.model.model
    assert inner.config.n_layer == 2 and inner.config.vocab_size == len(tok)      # vocabulary is ours
    hsd = hf.state_dict()
    for k in ("transformer.wpe.weight", "transformer.h.1.mlp.c_fc.weight", "transformer.h.0.attn.c_attn.bias",
              "transformer.ln_f.weight"):
        assert torch.equal(inner.state_dict()[k], hsd[k]), k
    wte = inner.transformer.wte.weight
    assert wte.shape == (len(tok), 64)
    assert abs(wte.mean().item() - hsd["transformer.wte.weight"].mean().item()) < 0.02
    assert abs(wte.std().item() / hsd["transformer.wte.weight"].std().item() - 1) < 0.1
    assert inner.lm_head.weight.data_ptr() == wte.data_ptr()                      # still tied
    # the same weights found through the Hugging Face cache layout when base_model is a name
    import shutil

    snap = tmp_path / "hf" / "hub" / "models--gpt2" / "snapshots" / "abc123"
    shutil.copytree(tmp_path / "gpt2-local", snap)
    os.environ["HF_HOME"] = str(tmp_path / "hf")
    try:
        named = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, use_pretrained=True,
                                 n_layer=2, n_embd=64, n_head=2, n_positions=64)
    finally:
        del os.environ["HF_HOME"]
    assert torch.equal(named.model.model.state_dict()["transformer.h.1.mlp.c_fc.weight"],
                       hsd["transformer.h.1.mlp.c_fc.weight"])


def test_checkpoints_with_wrapper_prefixes_and_mask_buffers_load():
    from allie_b200.models import load_model_state

    tok, ours, _ = _models()
    sd = {("_orig_mod." + k): v.clone() for k, v in ours.state_dict().items()}
    sd["_orig_mod.model.model.transformer.h.0.attn.bias"] = torch.ones(1, 1, 64, 64)
    sd["_orig_mod.model.model.transformer.h.0.attn.masked_bias"] = torch.tensor(-1e4)
    with torch.no_grad():
        for p in ours.parameters():
            p.zero_()
    load_model_state(ours, sd)
    assert float(ours.state_dict()["model.model.transformer.wte.weight"].abs().sum()) > 0
    sd.pop("_orig_mod.value_head.0.weight")
    with pytest.raises(RuntimeError):
        load_model_state(ours, sd)                # a missing parameter is still an error
