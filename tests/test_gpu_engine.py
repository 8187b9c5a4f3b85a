"""The layer-sliding engine around the GPU optimizer (SlideFormerOffloader).

What is checked
  * the loss equals a plain forward of the same Hugging Face model (same bf16 weights);
  * the gradients the engine hands to the optimizer match plain autograd gradients;
  * after each step every unit's fp32 weights, moments and bf16 weights equal the CPU oracle
    applied to exactly those gradients, bit for bit (one reference call per 32 Mi-element chunk);
  * host-resident state, host activation offload and no-checkpoint modes give the same bits as
    the default mode; tied embeddings (GPT-2) train the shared weight once.
"""
import copy

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def _bits(t):
    return t.detach().float().cpu().numpy().view(np.uint32) if t.dtype == torch.float32 else \
        t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def _make(name, **kw):
    from slideformer_b200.model_compat import build_random_model
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    model = build_random_model(name, DEV, torch.bfloat16, seed=3)
    plain = copy.deepcopy(model)
    eng = SlideFormerOffloader(model, DEV, torch.bfloat16, enable_timing=False, enable_memory_stats=False,
                               optimizer_kwargs=dict(HP), auto_backward_in_forward=False, **kw)
    return eng, plain


def _capture_grads(eng):
    """Copy each unit's flat gradient right before its optimizer step."""
    grabbed = {}
    for u in eng.transformer_layers:
        orig = u.update_params

        def wrapped(u=u, orig=orig):
            if u._unit is not None:
                grabbed[u.layer_idx] = u._unit["grad"][: u.total_size].clone()
            return orig()
        u.update_params = wrapped
    return grabbed


def _run_steps(eng, ids_list, oracle, check_plain=None):
    from oracle import oracle as O  # noqa: F401
    n_units = len(eng.transformer_layers)
    cpu = {}
    for u in eng.transformer_layers:
        n = u.total_size
        cpu[u.layer_idx] = [u._params_flat.detach().cpu().numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32),
                            np.zeros(n, np.uint16)]
    orc = oracle.OracleAdam(HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"], True)
    grabbed = _capture_grads(eng)
    losses = []
    for step, ids in enumerate(ids_list, start=1):
        grabbed.clear()
        if check_plain is not None and step == 1:
            plain_out = check_plain(input_ids=ids, labels=ids)
            plain_out.loss.backward()
        out = eng(ids, labels=ids)
        out.loss.backward()
        eng.wait_for_completion()
        losses.append(float(out.loss.detach()))
        if check_plain is not None and step == 1:
            assert abs(float(plain_out.loss) - losses[0]) < 2e-2 * abs(float(plain_out.loss)), (float(plain_out.loss), losses[0])
        assert sorted(grabbed) == list(range(n_units)), f"units updated: {sorted(grabbed)}"
        # the optimizer stream consumes units in backward order: output unit first, embedding last
        for idx in range(n_units - 1, -1, -1):
            u = eng.transformer_layers[idx]
            g = grabbed[idx].view(torch.int16).cpu().numpy().view(np.uint16)
            p, m, v, o = cpu[idx]
            for cs in range(0, u.total_size, u.update_chunk):
                ce = min(cs + u.update_chunk, u.total_size)
                orc.adam_update(step, HP["lr"], *HP["betas"], HP["eps"], HP["weight_decay"], True,
                                p[cs:ce], g[cs:ce], m[cs:ce], v[cs:ce], o[cs:ce])
    for idx in range(n_units):
        u = eng.transformer_layers[idx]
        p, m, v, o = cpu[idx]
        assert np.array_equal(_bits(u._params_flat.to(DEV)), p.view(np.uint32)), f"unit {idx} p"
        assert np.array_equal(_bits(eng.layer_optimizer.exp_avg_flat[idx].to(DEV)), m.view(np.uint32)), f"unit {idx} m"
        assert np.array_equal(_bits(eng.layer_optimizer.exp_avg_sq_flat[idx].to(DEV)), v.view(np.uint32)), f"unit {idx} v"
        assert np.array_equal(_bits(u._bf16_flat), o), f"unit {idx} bf16"
        # the module's live parameters ARE the bf16 weights
        name, prm = u._managed_named_params[0]
        off, shape, k = u._param_maps[name]
        assert prm.data.data_ptr() == u._bf16_flat[off:off + k].data_ptr()
    return losses, grabbed


def _ids(vocab, batch, seq, n, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=gen).to(DEV) for _ in range(n)]


@pytest.mark.parametrize("name", ["llama-tiny", "gpt2-tiny"])
def test_engine_steps_match_oracle_and_plain_model(name, oracle):
    eng, plain = _make(name)
    vocab = eng.config.vocab_size
    ids = _ids(vocab, 2, 32, 3)
    losses, grabbed = _run_steps(eng, ids, oracle, check_plain=plain)
    assert all(np.isfinite(losses))
    assert losses[-1] < losses[0] + 0.5
    # gradients of the last step vs plain autograd on a model holding the engine's weights of that step
    # (step 1 comparison): rerun step-1 gradients on the plain copy
    eng2, plain2 = _make(name)
    g2 = _capture_grads(eng2)
    out = eng2(ids[0], labels=ids[0])
    out.loss.backward()
    eng2.wait_for_completion()
    plain2.zero_grad()
    plain2(input_ids=ids[0], labels=ids[0]).loss.backward()
    named = dict(plain2.named_parameters())
    for u in eng2.transformer_layers[1:-1]:
        flat = g2[u.layer_idx].float()
        prefix = ("model.layers." if name.startswith("llama") else "transformer.h.") + f"{u.layer_idx - 1}."
        for pname, (off, shape, k) in u._param_maps.items():
            ref = named[prefix + pname].grad.float().reshape(-1)
            got = flat[off:off + k]
            denom = ref.norm().item() + 1e-12
            assert (got - ref).norm().item() / denom < 5e-2, (u.layer_idx, pname)


def test_tied_embedding_is_owned_once():
    eng, _ = _make("gpt2-tiny")
    assert eng.is_tied
    wte = eng.parts.embed.wte.weight
    assert eng.parts.lm_head.weight is wte
    assert any(p is wte for _, p in eng.embed_layer._managed_named_params)
    assert not any(p is wte for _, p in eng.output_layer._managed_named_params)
    total = sum(u.total_size for u in eng.transformer_layers)
    assert total == sum(p.numel() for p in eng.base_model.parameters())


@pytest.mark.parametrize("kw", [dict(state_device="host"), dict(activation_offload="host"),
                                dict(activation_checkpoint=False), dict(double_buffer=True),
                                dict(update_chunk=4096)])
def test_engine_modes_agree_bitwise(kw, oracle):
    base, _ = _make("llama-tiny")
    other, _ = _make("llama-tiny", **kw)
    # a different chunking is a different reference call sequence (pow() vs running product for
    # beta^t), so it is compared after one step, before the weights can drift apart
    ids = _ids(base.config.vocab_size, 2, 32, 1 if "update_chunk" in kw else 3, seed=9)
    for e in (base, other):
        for x in ids:
            e(x, labels=x).loss.backward()
            e.wait_for_completion()
    for ub, uo in zip(base.transformer_layers, other.transformer_layers):
        if "update_chunk" in kw:
            # within the specified 2-ulp budget
            a, b = ub._params_flat.cpu().numpy(), uo._params_flat.cpu().numpy()
            assert np.max(np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))) <= 2
        else:
            assert np.array_equal(_bits(ub._params_flat.to(DEV)), _bits(uo._params_flat.to(DEV))), ub.layer_idx
            assert np.array_equal(_bits(ub._bf16_flat), _bits(uo._bf16_flat))
    if kw.get("activation_offload") == "host":
        st = other.activation_store
        assert st is not None and st.bytes_d2h > 0 and st.bytes_h2d > 0


def test_host_state_keeps_the_reference_call_history_per_chunk(oracle):
    """Units larger than the update chunk: the reference engine makes one adam_update per chunk
    (transformer_layer.py:453-499), so from the second chunk on beta^t comes from pow().  The
    host-resident mode must follow that history like the HBM-resident mode does: equal bits with
    the same chunk size, over several steps, and both equal to the oracle called once per chunk
    (checked inside _run_steps)."""
    hbm, _ = _make("llama-tiny", update_chunk=4096)
    host, _ = _make("llama-tiny", update_chunk=4096, state_device="host")
    ids = _ids(hbm.config.vocab_size, 2, 32, 3, seed=4)
    _run_steps(hbm, ids, oracle)
    _run_steps(host, ids, oracle)
    assert any(u.total_size > 2 * 4096 for u in host.transformer_layers)
    for ub, uo in zip(hbm.transformer_layers, host.transformer_layers):
        assert np.array_equal(_bits(ub._params_flat.to(DEV)), _bits(uo._params_flat.to(DEV))), ub.layer_idx
        assert np.array_equal(_bits(ub._bf16_flat), _bits(uo._bf16_flat))


def _train(eng, ids):
    for x in ids:
        eng(x, labels=x).loss.backward()
        eng.wait_for_completion()


@pytest.mark.parametrize("kw", [dict(weight_window=True), dict(weight_window=True, state_device="host"),
                                dict(weight_window=True, double_buffer=True)])
def test_one_gpu_weight_window_matches_resident_weights(kw, tmp_path):
    """bf16 weights parked in pinned host memory and copied into a 2- or 3-unit window one unit
    ahead (the reference's headline mode, offload_transformer.py:75-79): same bits as keeping
    every layer's bf16 weights in HBM, and no unit holds a device-resident copy."""
    base, _ = _make("llama-tiny")
    win, _ = _make("llama-tiny", **kw)
    ids = _ids(base.config.vocab_size, 2, 32, 3, seed=12)
    _train(base, ids)
    _train(win, ids)
    for ub, uw in zip(base.transformer_layers, win.transformer_layers):
        assert uw._bf16_flat is None and uw._bf16_host.is_pinned()
        assert np.array_equal(_bits(ub._params_flat.to(DEV)), _bits(uw._params_flat.to(DEV))), ub.layer_idx
        assert np.array_equal(_bits(ub._bf16_flat), _bits(uw.bf16_weights_flat().to(DEV))), ub.layer_idx
    # inference after training uses the window too
    with torch.no_grad():
        a, b = base(ids[0]).logits.float(), win(ids[0]).logits.float()
    assert torch.equal(a, b)
    from transformers import AutoModelForCausalLM
    out = win.save_pretrained(str(tmp_path / "ckpt"))
    again = AutoModelForCausalLM.from_pretrained(out, dtype=torch.bfloat16).to(DEV)
    with torch.no_grad():
        assert (again(input_ids=ids[0]).logits.float() - a).abs().max().item() < 0.1


def test_auto_state_placement_splits_units_between_hbm_and_host():
    """state_device='auto' with a small HBM budget: the first units keep their fp32 state in HBM,
    the rest stream it from pinned host memory; the result has the bits of the all-HBM run."""
    from slideformer_b200.offload_transformer import plan_state_placement, unit_numels
    base, _ = _make("llama-tiny")
    sizes = unit_numels(base.parts)
    assert sizes == [u.total_size for u in base.transformer_layers]
    budget = 12 * (sizes[0] + sizes[1]) + 100     # the embedding and the first decoder layer fit
    auto, _ = _make("llama-tiny", state_device="auto", hbm_state_budget_gb=budget / 2 ** 30)
    want = plan_state_placement(sizes, budget)
    assert want[:2] == ["hbm", "hbm"] and "host" in want
    assert [u.state_device for u in auto.transformer_layers] == want
    for u in auto.transformer_layers:
        assert u._params_flat.is_cuda == (u.state_device == "hbm")
        assert auto.layer_optimizer.exp_avg_flat[u.layer_idx].is_cuda == (u.state_device == "hbm")
    ids = _ids(base.config.vocab_size, 2, 32, 3, seed=13)
    _train(base, ids)
    _train(auto, ids)
    for ub, ua in zip(base.transformer_layers, auto.transformer_layers):
        assert np.array_equal(_bits(ub._params_flat.to(DEV)), _bits(ua._params_flat.to(DEV))), ub.layer_idx
        assert np.array_equal(_bits(ub._bf16_flat), _bits(ua._bf16_flat))


def test_timer_labels_and_stats(capsys):
    """Every label of the reference's timer that has a counterpart here gets samples
    (utils/timer.py:11-21), and print_layer_stats prints them in the reference's format."""
    from slideformer_b200.model_compat import build_random_model
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    model = build_random_model("llama-tiny", DEV, torch.bfloat16, seed=3)
    eng = SlideFormerOffloader(model, DEV, torch.bfloat16, enable_timing=True, optimizer_kwargs=dict(HP),
                               auto_backward_in_forward=False, activation_offload="host", weight_window=True)
    ids = _ids(eng.config.vocab_size, 2, 32, 2, seed=14)
    _train(eng, ids)
    stats = eng.layer_timings_ms()
    n_units = len(eng.transformer_layers)
    for op in ("forward", "backward", "parameter_update", "h2d_transfer_fw", "h2d_transfer_bw", "ac_fwd_d2h", "ac_bwd_h2d"):
        assert op in stats and all(ms >= 0 for _, ms, _ in stats[op]), op
    assert len(stats["forward"]) == n_units and len(stats["parameter_update"]) == n_units
    assert eng.parameter_update_ms().keys() == set(range(n_units))
    eng.print_layer_stats()
    eng.print_layer_stats(show_history=True)
    eng.print_layer_stats(layer_idx=1)
    text = capsys.readouterr().out
    for label in ("Current Step Layer Statistics:", "Historical Average Layer Statistics:", "  forward: ", "  backward: ",
                  "  parameter update: ", "  h2d transfer fw: ", "  ac fwd d2h: ", "  ac bwd h2d: ", "avg across", "avg over"):
        assert label in text, label


def test_engine_grad_stats_match_the_gradients_it_consumed():
    """sum(g*g) gathered inside the update kernels equals the norm of the flat gradients the engine
    handed to the optimizer, and a multiplier of 1/2 halves the first step's Adam moments."""
    eng, _ = _make("llama-tiny")
    eng.enable_grad_stats()
    grabbed = _capture_grads(eng)
    ids = _ids(eng.config.vocab_size, 2, 32, 1, seed=21)[0]
    eng(ids, labels=ids).loss.backward()
    st = eng.read_grad_stats()
    want = sum(float(g.float().double().pow(2).sum()) for g in grabbed.values())
    assert st["nonfinite"] is False and st["sumsq"] == pytest.approx(want, rel=1e-4)
    assert eng.clip_scale_for_next_step(st["norm"] * 0.5, st) == pytest.approx(0.5)
    assert eng.clip_scale_for_next_step(st["norm"] * 2.0, st) == 1.0
    half, _ = _make("llama-tiny")
    half.set_grad_scale(0.5)
    half(ids, labels=ids).loss.backward()
    half.wait_for_completion()
    m_full = eng.layer_optimizer.exp_avg_flat[1]
    m_half = half.layer_optimizer.exp_avg_flat[1]
    assert torch.allclose(m_half * 2, m_full, rtol=1e-6, atol=1e-30)   # m = (1 - beta1) * g after one step; halving g is exact


def test_close_releases_the_engine_memory():
    """Autograd holds the gradient hooks where the cycle collector cannot see them; close() is what
    returns an engine's HBM (a benchmark that builds several engines in one process needs it)."""
    import gc
    before = None
    for kw in (dict(), dict(), dict(state_device="host"), dict(weight_window=True, activation_offload="host")):
        if before is None:
            # the first engine of a process also brings up library workspaces that stay: measure from here
            warm, _ = _make("llama-tiny")
            x = _ids(warm.config.vocab_size, 2, 32, 1)[0]
            warm(x, labels=x).loss.backward()
            warm.close()
            del warm, x, _
            gc.collect()
            torch.cuda.empty_cache()
            before = torch.cuda.memory_allocated()
        eng, plain = _make("llama-tiny", **kw)
        del plain
        ids = _ids(eng.config.vocab_size, 2, 32, 1)[0]
        eng(ids, labels=ids).loss.backward()
        eng.wait_for_completion()
        assert torch.cuda.memory_allocated() - before > (256 << 10)
        eng.close()
        eng.close()                      # idempotent
        del eng, ids
        gc.collect()
        torch.cuda.empty_cache()
        assert torch.cuda.memory_allocated() - before < (64 << 10), kw


def test_inference_forward_and_lr_update():
    eng, plain = _make("llama-tiny")
    ids = _ids(eng.config.vocab_size, 2, 16, 1)[0]
    with torch.no_grad():
        logits = eng(ids).logits
        ref = plain(input_ids=ids).logits
    assert logits.shape == ref.shape
    assert (logits.float() - ref.float()).abs().max().item() < 0.1
    eng.update_learning_rate(5e-4)
    assert eng.layer_optimizer.defaults["lr"] == 5e-4
    assert all(g["lr"] == 5e-4 for g in eng.layer_optimizer.param_groups)


def test_save_pretrained_round_trip(tmp_path):
    """Weights written after a step reload into a plain Hugging Face model that gives the engine's logits."""
    from transformers import AutoModelForCausalLM
    eng, _ = _make("llama-tiny")
    ids = _ids(eng.config.vocab_size, 2, 16, 1)[0]
    eng(ids, labels=ids).loss.backward()
    eng.wait_for_completion()
    out = eng.save_pretrained(str(tmp_path / "ckpt"))
    reloaded = AutoModelForCausalLM.from_pretrained(out, dtype=torch.bfloat16).to(DEV)
    with torch.no_grad():
        a = eng(ids).logits.float()
        b = reloaded(input_ids=ids).logits.float()
    assert torch.allclose(a, b, atol=2e-2, rtol=0), (a - b).abs().max().item()


def test_host_grad_stepper_matches_oracle(oracle):
    """The chunked host-gradient pipeline (pinned bf16 gradient in, pinned bf16 weights out)."""
    from slideformer_b200 import LayerAdam
    from slideformer_b200.host_io import HostGradStepper
    n, chunk = 5 * 4096 + 48, 4096
    hp = (HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"])
    gen = torch.Generator().manual_seed(4)
    p0 = torch.randn(n, generator=gen) * 0.02
    po, mo, vo, oo = p0.numpy().copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), np.zeros(n, np.uint16)
    pd, md, vd = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    od = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    out_host = torch.zeros(n, dtype=torch.bfloat16).pin_memory()
    opt = LayerAdam(**HP)
    orc = oracle.OracleAdam(*hp, True)
    stepper = HostGradStepper(opt, n, DEV, chunk_numel=chunk, min_chunk_numel=256)
    assert stepper.chunks[0] == (0, 256) and stepper.chunks[-1][1] == n and len(stepper.chunks) > 6
    group = dict(opt.defaults, step=0)
    for step in (1, 2, 3):
        g = (torch.randn(n, generator=gen) * 1e-3).to(torch.bfloat16)
        gnp = g.view(torch.int16).numpy().view(np.uint16)
        for cs, ce in stepper.chunks:   # one reference call per piece, like the reference's chunk consumer
            orc.adam_update(step, *hp, True, po[cs:ce], gnp[cs:ce], mo[cs:ce], vo[cs:ce], oo[cs:ce])
        group["step"] = step
        # steps 1 and 2 are left to overlap; the last one is joined
        stepper.step(pd, g.pin_memory(), md, vd, od, out_host, dict(group), join=(step == 3))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(pd), po.view(np.uint32))
    assert np.array_equal(_bits(md), mo.view(np.uint32)) and np.array_equal(_bits(vd), vo.view(np.uint32))
    assert np.array_equal(out_host.view(torch.int16).numpy().view(np.uint16), oo)


def test_layer_stats_and_csv(tmp_path, capsys):
    from slideformer_b200.finetune_bench import append_result_to_csv, run_finetune
    line = run_finetune("llama-tiny", 2, 32, steps=2, warmup=1, dev=DEV)
    assert line["value"] > 0 and line["gpu_launches"] == 2 * 5 and line["optimizer_ms_per_step"] > 0
    append_result_to_csv(str(tmp_path / "r.csv"), line)
    rows = (tmp_path / "r.csv").read_text().splitlines()
    assert rows[0].startswith("Model,Sequence_Length") and rows[1].startswith("llama-tiny,32,2,bf16,1,hbm")
    from slideformer_b200.model_compat import build_random_model
    from slideformer_b200.offload_transformer import SlideFormerOffloader
    eng = SlideFormerOffloader(build_random_model("llama-tiny", DEV), DEV, torch.bfloat16, enable_timing=True,
                               enable_memory_stats=False, optimizer_kwargs=dict(HP))
    ids = _ids(eng.config.vocab_size, 2, 16, 1)[0]
    eng(ids, labels=ids)
    eng.print_layer_stats()
    eng.print_layer_stats(layer_idx=1, show_history=True)
    out = capsys.readouterr().out
    assert "Current Step Layer Statistics" in out and "parameter update" in out and "Layer 1 Statistics" in out
