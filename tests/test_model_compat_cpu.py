"""Model glue on the CPU: unit layout, tie detection, size bookkeeping, per-layer inputs,
meta-device skeletons.  No CUDA needed."""
import pytest
import torch

from slideformer_b200.model_compat import (MODEL_SPECS, build_random_model, call_decoder_layer, parameter_sizes,
                                            prepare_layer_inputs, split_parts, validate_model)


@pytest.mark.parametrize("name,tied", [("llama-tiny", False), ("gpt2-tiny", True)])
def test_parts_and_sizes(name, tied):
    model = build_random_model(name, "cpu", torch.float32, seed=1)
    parts = validate_model(model)
    assert (parts.tied_param is not None) == tied
    assert len(parts.layers) == (3 if name == "llama-tiny" else 2)
    max_unit, total = parameter_sizes(model)
    assert total == sum(p.numel() for p in model.parameters())
    unit_sizes = [sum(p.numel() for p in m.parameters()) for m in (parts.embed, *parts.layers)]
    assert max_unit >= max(unit_sizes)
    ids = torch.randint(0, model.config.vocab_size, (2, 12))
    h = parts.embed(ids)
    kwargs = prepare_layer_inputs(parts, h)
    assert len(kwargs) == len(parts.layers) and kwargs[0]["attention_mask"] is None
    out = call_decoder_layer(parts.layers[0], h, kwargs[0])
    assert out.shape == h.shape
    # a padding mask produces a real mask
    mask = torch.ones(2, 12, dtype=torch.bool)
    mask[1, 8:] = False
    assert prepare_layer_inputs(parts, h, attention_mask=mask)[0]["attention_mask"] is not None


def test_layered_forward_equals_model_forward():
    model = build_random_model("llama-tiny", "cpu", torch.float32, seed=2).eval()
    parts = split_parts(model)
    ids = torch.randint(0, model.config.vocab_size, (2, 10))
    with torch.no_grad():
        h = parts.embed(ids)
        for layer, kw in zip(parts.layers, prepare_layer_inputs(parts, h)):
            h = call_decoder_layer(layer, h, kw)
        logits = parts.lm_head(parts.norm(h))
        ref = model(input_ids=ids).logits
    assert torch.allclose(logits, ref, atol=1e-5)


def test_gpt2_embedding_unit_adds_positions():
    model = build_random_model("gpt2-tiny", "cpu", torch.float32, seed=3).eval()
    parts = split_parts(model)
    ids = torch.randint(0, model.config.vocab_size, (1, 9))
    with torch.no_grad():
        h = parts.embed(ids)
        for layer, kw in zip(parts.layers, prepare_layer_inputs(parts, h)):
            h = call_decoder_layer(layer, h, kw)
        logits = parts.lm_head(parts.norm(h))
        ref = model(input_ids=ids).logits
    assert torch.allclose(logits, ref, atol=1e-4)


def test_meta_skeleton_has_no_storage_but_real_rotary():
    model = build_random_model("llama-tiny", "cpu", torch.bfloat16, meta=True)
    assert all(p.is_meta for p in model.parameters())
    parts = validate_model(model)
    assert not parts.rotary_emb.inv_freq.is_meta
    big = MODEL_SPECS["llama3.1-70b"]
    assert big["num_hidden_layers"] == 80 and big["hidden_size"] == 8192


def test_benchmark_layer_size_is_the_llama_8b_decoder_layer():
    spec = MODEL_SPECS["llama3.1-8b"]
    h, kv, inter = spec["hidden_size"], spec["num_key_value_heads"] * (spec["hidden_size"] // spec["num_attention_heads"]), spec["intermediate_size"]
    n = 2 * h * h + 2 * h * kv + 3 * h * inter + 2 * h
    assert n == 218_112_000


def test_chunk_schedule_covers_the_range_with_short_ends():
    from slideformer_b200.host_io import chunk_schedule
    for n, c, m in ((218_112_000, 16 << 20, 1 << 20), (20528, 4096, 256), (100, 4096, 16), (163847, 4096, 64), (1 << 20, 1 << 18, 1 << 14)):
        p = chunk_schedule(n, c, m)
        assert p[0][0] == 0 and p[-1][1] == n
        assert all(a < b and a % 16 == 0 and b - a <= c for a, b in p)
        assert all(p[i][1] == p[i + 1][0] for i in range(len(p) - 1))
    p = chunk_schedule(218_112_000, 16 << 20, 1 << 20)
    assert p[0][1] - p[0][0] == 1 << 20 and p[-1][1] - p[-1][0] == 1 << 20 and len(p) == 20
    with pytest.raises(ValueError):
        chunk_schedule(100, 24, 8)
