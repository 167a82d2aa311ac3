"""End-to-end numerics of the native (bf16, fused kernels) training path against the plain PyTorch fp32 path of the
same model: loss, every parameter gradient, and a short training curve."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _config(layers=2, hidden=256, heads=4, kv=2, inter=512, vocab=1024, moe=False):
    from lm_engine.hf_models import GPTBaseConfig

    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=inter, add_bias=False)
    return GPTBaseConfig(
        vocab_size=vocab, hidden_size=hidden, num_layers=layers, max_position_embeddings=1024, position_embedding_type="rope",
        normalization_function="rmsnorm", tie_word_embeddings=False,
        sequence_mixer_blocks=[dict(sequence_mixer_type="softmax_attention", num_attention_heads=heads, num_key_value_heads=kv, add_bias=False)] * layers,
        mlp_blocks=[dict(mlp)] * layers,
    )


def _all_kernels():
    from lm_engine.enums import Kernel

    return [k for k in Kernel if k != Kernel.ladder_residual_overlapped_layer]


def _build_pair(config):
    from lm_engine.hf_models import GPTBaseForCausalLM
    from lm_engine.parallel.engine import ShardedTrainingEngine

    torch.manual_seed(0)
    device = torch.device("cuda", 0)
    reference = GPTBaseForCausalLM(config, use_padding_free_transformer=True).to(device)
    model = GPTBaseForCausalLM(config, use_padding_free_transformer=True)
    model.load_state_dict(reference.state_dict())
    engine = ShardedTrainingEngine(model, compute_dtype=torch.bfloat16, device=device)
    model._lm_engine = engine
    return reference, model, engine


@pytest.mark.parametrize("heads,kv,hidden", [(4, 2, 256), (2, 2, 256), (4, 1, 512)])
def test_native_gradients_match_fp32_reference(heads, kv, hidden):
    from lm_engine import ops
    from lm_engine.kernels import enable_kernels

    config = _config(hidden=hidden, heads=heads, kv=kv)
    reference, model, engine = _build_pair(config)
    docs = [torch.randint(0, 1024, (n,)).tolist() for n in (300, 129, 64, 411)]

    ref_out = reference(input_ids=docs, labels=docs, reduction="sum")
    ref_out.loss.backward()
    with enable_kernels(_all_kernels()):
        out = model(input_ids=docs, labels=docs, reduction="sum")
        out.loss.backward()
        engine.fold_autograd_grads()
    torch.cuda.synchronize()
    ops.check_status()
    assert abs(float(out.loss) - float(ref_out.loss)) < 1e-2 * abs(float(ref_out.loss))

    ref_grads = dict(reference.named_parameters())
    worst = 0.0
    for name, p in model.named_parameters():
        g = p.main_grad.float()
        r = ref_grads[name].grad.float()
        err = ((g - r).norm() / (r.norm() + 1e-12)).item()
        worst = max(worst, err)
        assert err < 6e-2, f"{name}: relative gradient error {err}"
    assert worst > 0  # the two paths are different code


def test_native_training_curve_tracks_fp32_reference():
    from lm_engine import ops
    from lm_engine.kernels import enable_kernels
    from lm_engine.optimization import build_optimizer

    config = _config()
    reference, model, engine = _build_pair(config)
    opt_args = dict(lr=1e-3, weight_decay=0.1, betas=[0.9, 0.95], eps=1e-10)
    optimizer = build_optimizer(model, "TorchAdamW", opt_args, None)
    ref_opt = torch.optim.AdamW(reference.parameters(), lr=1e-3, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-10)
    # weight decay groups differ (norm weights are exempt in the engine): exempt them in the reference too
    decay = [p for n, p in reference.named_parameters() if "ln_" not in n]
    no_decay = [p for n, p in reference.named_parameters() if "ln_" in n]
    ref_opt = torch.optim.AdamW([{"params": decay}, {"params": no_decay, "weight_decay": 0.0}], lr=1e-3, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-10)

    gen = torch.Generator().manual_seed(1)
    curve, ref_curve = [], []
    for _ in range(8):
        docs = [torch.randint(0, 1024, (n,), generator=gen).tolist() for n in (256, 200, 120)]
        ref_loss = reference(input_ids=docs, labels=docs, reduction="mean").loss
        ref_opt.zero_grad()
        ref_loss.backward()
        torch.nn.utils.clip_grad_norm_(reference.parameters(), 1.0)
        ref_opt.step()
        with enable_kernels(_all_kernels()):
            loss = model(input_ids=docs, labels=docs, reduction="mean").loss
            loss.backward()
            engine.fold_autograd_grads()
        engine.optimizer_step(optimizer, None, 1.0)
        curve.append(float(loss))
        ref_curve.append(float(ref_loss))
    ops.check_status()
    for a, b in zip(curve, ref_curve):
        assert abs(a - b) < 3e-2 * abs(b), (curve, ref_curve)
    assert all(abs(v) < 20 for v in curve)


@pytest.mark.parametrize("side", ["none", "left", "right"])
def test_padded_batches_run_on_the_varlen_kernels(side):
    """A padded [batch, seq] batch (no mask, left padding, right padding) through pack -> variable-length attention
    kernels -> unpack gives the logits of the masked dense attention at every real position."""
    from lm_engine.hf_models import GPTBaseForCausalLM
    from lm_engine.kernels import enable_kernels

    torch.manual_seed(0)
    device = torch.device("cuda", 0)
    model = GPTBaseForCausalLM(_config(), use_padding_free_transformer=False).to(device=device, dtype=torch.bfloat16).eval()
    batch, seq = 3, 200
    ids = torch.randint(0, 1024, (batch, seq), device=device)
    lengths = [200, 131, 64]
    mask = None
    if side != "none":
        mask = torch.zeros(batch, seq, dtype=torch.long, device=device)
        for i, n in enumerate(lengths):
            if side == "left":
                mask[i, seq - n:] = 1
            else:
                mask[i, :n] = 1
    with torch.no_grad():
        ref = model(input_ids=ids, attention_mask=mask).logits.float()
        from lm_engine.enums import Kernel

        with enable_kernels([k for k in _all_kernels() if k != Kernel.fused_linear_cross_entropy_cute]):
            got = model(input_ids=ids, attention_mask=mask).logits.float()
    keep = torch.ones(batch, seq, dtype=torch.bool, device=device) if mask is None else mask.bool()
    err = (got - ref)[keep].abs().max().item()
    assert err < 0.1 * ref[keep].abs().max().item() + 0.05, err


def test_recurrent_and_state_space_mixers_on_their_scan_kernels():
    """A model with Mamba-2, GRU and RNN mixers gives the same logits and parameter gradients with the scan kernels
    (SSD scan, depthwise convolution, GRU / RNN scans) as with the PyTorch formulations of the same layers."""
    from lm_engine.enums import Kernel
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.kernels import enable_kernels

    torch.manual_seed(0)
    device = torch.device("cuda", 0)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=256, add_bias=False)
    config = GPTBaseConfig(
        vocab_size=512, hidden_size=128, num_layers=3, max_position_embeddings=512, position_embedding_type="nope",
        normalization_function="rmsnorm",
        sequence_mixer_blocks=[
            dict(sequence_mixer_type="mamba2", state_size=64, intermediate_size=256, num_heads=4, conv_kernel_size=4, num_groups=2, chunk_size=64),
            dict(sequence_mixer_type="gru", state_size=128, num_heads=4, add_bias=False),
            dict(sequence_mixer_type="rnn", state_size=128, num_heads=2, add_bias=False),
        ],
        mlp_blocks=[dict(mlp)] * 3,
    )
    model = GPTBaseForCausalLM(config, use_padding_free_transformer=False).to(device)
    ids = torch.randint(0, 512, (2, 96), device=device)

    def run(kernels):
        model.zero_grad(set_to_none=True)
        with enable_kernels(kernels):
            out = model(input_ids=ids, labels=ids)
        out.loss.backward()
        return out.logits.detach().float(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}

    ref_logits, ref_grads = run([])
    logits, grads = run([Kernel.mamba2_ssm, Kernel.gru_cute, Kernel.rnn_cute, Kernel.causal_conv1d])
    assert (logits - ref_logits).abs().max().item() < 2e-3 * ref_logits.abs().max().item() + 1e-4
    assert set(grads) == set(ref_grads)
    for name, g in grads.items():
        r = ref_grads[name]
        assert (g - r).norm().item() <= 2e-3 * r.norm().item() + 1e-6, name


def test_packed_documents_through_the_scan_kernels_match_the_per_document_loops():
    """Padding-free batches: Mamba-2 (convolution + SSD scan with the state reset at document starts), GRU and RNN take
    the document boundaries from cu_seqlens inside the kernels; the result equals running every document on its own."""
    from lm_engine.enums import Kernel
    from lm_engine.hf_models import GPTBaseConfig, GPTBaseForCausalLM
    from lm_engine.kernels import enable_kernels

    torch.manual_seed(0)
    device = torch.device("cuda", 0)
    mlp = dict(mlp_type="MLP", activation_function="swiglu", intermediate_size=256, add_bias=False)
    config = GPTBaseConfig(
        vocab_size=512, hidden_size=128, num_layers=2, max_position_embeddings=512, position_embedding_type="nope",
        normalization_function="rmsnorm",
        sequence_mixer_blocks=[
            dict(sequence_mixer_type="mamba2", state_size=64, intermediate_size=256, num_heads=4, conv_kernel_size=4, num_groups=2, chunk_size=64),
            dict(sequence_mixer_type="gru", state_size=128, num_heads=4, add_bias=False),
        ],
        mlp_blocks=[dict(mlp)] * 2,
    )
    model = GPTBaseForCausalLM(config, use_padding_free_transformer=True).to(device)
    docs = [torch.randint(0, 512, (n,)).tolist() for n in (70, 3, 129, 40)]

    def run(kernels):
        model.zero_grad(set_to_none=True)
        with enable_kernels(kernels):
            out = model(input_ids=docs, labels=docs)
        out.loss.backward()
        return out.logits.detach().float(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}

    ref_logits, ref_grads = run([])
    logits, grads = run([Kernel.mamba2_ssm, Kernel.gru_cute, Kernel.causal_conv1d])
    assert (logits - ref_logits).abs().max().item() < 2e-3 * ref_logits.abs().max().item() + 1e-4
    for name, g in grads.items():
        r = ref_grads[name]
        assert (g - r).norm().item() <= 3e-3 * r.norm().item() + 1e-6, name


def test_cpu_offload_keeps_masters_on_the_host_and_trains_the_same(tmp_path):
    """``distributed_args.cpu_offload`` on a GPU: the fp32 master shards and the optimizer's moments sit in pinned host
    memory, the optimizer runs on the CPU, and the loss curve equals the one of the run that keeps them on the device."""
    import json
    import os
    import subprocess
    import sys

    script = os.path.join(os.path.dirname(__file__), "scripts", "tiny_pretrain.py")
    curves = []
    for offload in (False, True):
        out = tmp_path / f"curve_{int(offload)}.json"
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29691", TINY_CPU_OFFLOAD="1" if offload else "0",
                   TINY_REPORT_STORAGE="1")
        subprocess.run([sys.executable, script, str(out), "8", "12", "3"], check=True, env=env, timeout=600, capture_output=True)
        curves.append(json.loads(out.read_text()))
    plain, offloaded = curves
    assert offloaded[-1].get("master_device") == "cpu" and offloaded[-1].get("optimizer_state_device") == "cpu"
    assert plain[-1].get("master_device", "cuda").startswith("cuda")
    for a, b in zip(plain, offloaded):
        assert abs(a["loss"] - b["loss"]) < 1e-4 * max(1.0, abs(a["loss"]))
        assert abs(a["grad_norm"] - b["grad_norm"]) < 1e-3 * max(1.0, abs(a["grad_norm"]))
