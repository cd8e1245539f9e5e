"""CPU checks of the decoder shape tables the partitioned benchmark workloads are built from: the linears per layer
and the parameter totals follow the reference's configurations (LlamaConfig::llama3_1b, src/llama.rs:64-80;
Qwen35Config::qwen35_9b and its per-layer parameter counts, src/qwen35.rs:70-102,146-197)."""
from helpers import PKG  # noqa: F401  (puts the package on sys.path)


def test_llama32_1b_linears():
    from alice_train import decoder_step as ds
    tokens, layers, std, guard = ds.MODELS["llama32-1b-qat"]()
    assert tokens == 8192 and len(layers) == 16
    shapes = {n: (o, i) for n, o, i in layers[0]}
    assert shapes == {"q_proj": (2048, 2048), "k_proj": (512, 2048), "v_proj": (512, 2048), "o_proj": (2048, 2048),
                      "gate_proj": (8192, 2048), "up_proj": (8192, 2048), "down_proj": (2048, 8192)}
    per_layer = sum(o * i for _, o, i in layers[0])
    assert per_layer == 60_817_408                      # 60.8 M ternary weights per layer
    assert 16 * per_layer * 4 == 3_892_314_112          # 3.89 GB of f32 dW per step


def test_qwen35_9b_linears():
    from alice_train import decoder_step as ds
    tokens, layers, std, guard = ds.MODELS["qwen35-9b-hybrid"]()
    assert tokens == 8192 and len(layers) == 32
    kinds = ["full" if any(n == "q_proj" for n, _, _ in layer) else "delta" for layer in layers]
    assert kinds.count("full") == 8 and all(kinds[i] == "full" for i in (3, 7, 11, 15, 19, 23, 27, 31))   # (i+1) % 4 == 0
    delta = {n: (o, i) for n, o, i in layers[0]}
    assert delta["in_proj_qkv"] == (8192, 4096) and delta["in_proj_z"] == (4096, 4096)
    assert delta["in_proj_b"] == (32, 4096) and delta["in_proj_a"] == (32, 4096) and delta["out_proj"] == (4096, 4096)
    assert delta["gate_proj"] == (12288, 4096) and delta["down_proj"] == (4096, 12288)
    full = {n: (o, i) for n, o, i in layers[3]}
    assert full["q_proj"] == (4096, 4096) and full["k_proj"] == (1024, 4096) and full["o_proj"] == (4096, 4096)
    # the linear part of deltanet_params_per_layer / full_attn_params_per_layer
    hidden, inter = 4096, 12288
    assert sum(o * i for _, o, i in layers[0]) == hidden * (2 * 2048 + 4096) + hidden * 4096 + 2 * hidden * 32 + 4096 * hidden + 3 * inter * hidden
    assert sum(o * i for _, o, i in layers[3]) == 2 * hidden * 4096 + 2 * hidden * 1024 + 3 * inter * hidden


def test_every_dw_is_divisible_for_the_in_switch_sum():
    from alice_train import decoder_step as ds
    for name in ("llama32-1b-qat", "qwen35-9b-hybrid"):
        _, layers, _, _ = ds.MODELS[name]()
        for layer in layers:
            for _, o, i in layer:
                assert (o * i) % (4 * 8) == 0   # ab_dp_allreduce_start: a multiple of 4 * world floats, up to 8 GPUs
