"""Named shapes for the random-weights mode of the command line tools and the benchmark.
The numbers are what the respective config.json files hold; they are data for `LlamaConfig`,
not constants of the engine."""

PRESETS = {
    "tinyA": dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16, intermediate_size=176, max_position_embeddings=128,
                  rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "tinyB": dict(vocab_size=320, hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
                  num_key_value_heads=1, head_dim=32, intermediate_size=256, max_position_embeddings=256,
                  rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "tinyllama": dict(vocab_size=32000, hidden_size=2048, num_hidden_layers=22, num_attention_heads=32,
                      num_key_value_heads=4, intermediate_size=5632, max_position_embeddings=2048,
                      rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "llama2-7b": dict(vocab_size=32000, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, intermediate_size=11008, max_position_embeddings=4096,
                      rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, intermediate_size=14336, max_position_embeddings=8192,
                      rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False),
}



def _dopudra(width, vocab, positions, streams, blocks, heads, dim, ff, softmax_heads, softmax_kv, softmax_dim):
    """`blocks` times: three lightning layers (the last with a feed-forward), then one parallel layer."""
    decay = [1.0 - 2.0 ** -(1 + 7 * h / max(heads - 1, 1)) for h in range(heads)]
    light = {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "decay": decay}, "mlp": None}
    both = {"type": "parallel", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"left": {"heads": softmax_heads, "kv_heads": softmax_kv, "dim": softmax_dim, "vdim": softmax_dim,
                               "conv": 4, "scale": softmax_dim ** -0.5, "bias_max": positions // 2, "bias_rows": 32,
                               "q_temp": {"coef": 0.1, "every": 128}},
                      "right": {"heads": heads, "dim": dim, "vdim": dim, "tau": 16.0, "rank": 32},
                      "left_scale": 1.0, "right_scale": 1.0}}
    layers = []
    for _ in range(blocks):
        layers += [light, light, dict(light, mlp={"kind": "dense", "ff": ff}), both]
    return dict(architecture="Dopudra", vocab=vocab, width=width, max_positions=positions, streams=streams,
                embedding={"scale": 1.0}, norm={"eps": 1e-6}, layers=layers)


PRESETS.update({
    "dopudra-tiny": _dopudra(64, 300, 512, 2, 1, 2, 16, 96, 2, 1, 32),
    # layer sizes near TinyLlama's (width 2048, feed-forward 5632, 32 heads of 64): 20 layers
    "dopudra-2048": _dopudra(2048, 32000, 4096, 4, 5, 32, 64, 5632, 32, 4, 64),
    # ... and near Llama-2-7B's (width 4096, 32 heads of 128): 32 layers
    "dopudra-4096": _dopudra(4096, 32000, 4096, 4, 8, 32, 128, 11008, 32, 32, 128),
})


def _zadurax(width, vocab, ff, heads, head_dim, kv_heads, window, latent_heads, latent_dim, rot_dim, kv_rank,
             state_heads, state_dim, repeats):
    """One layer of each mixer with a feed-forward, then `repeats` more runs of the three with the same tensors."""
    own = [{"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"heads": latent_heads, "dim": latent_dim, "rot_dim": rot_dim, "vdim": latent_dim, "kv_rank": kv_rank,
                      "scale": (latent_dim + rot_dim) ** -0.5,
                      "rot": {"base": 10000.0, "dims": rot_dim,
                              "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}},
           {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "mask": {"size": window},
                      "rot": {"base": 10000.0, "dims": head_dim // 2}, "scale": head_dim ** -0.5}},
           {"type": "mlstm", "mlp": {"kind": "dense", "ff": ff},
            "mixer": {"heads": state_heads, "dim": state_dim, "vdim": state_dim, "gate_cap": 15.0}}]
    layers = list(own)
    for _ in range(repeats):
        layers += [dict(layer, weights_of=j) for j, layer in enumerate(own)]
    return dict(architecture="Zadurax", vocab=vocab, width=width, norm={"eps": 1e-6}, layers=layers)


PRESETS.update({
    "zadurax-tiny": _zadurax(64, 300, 96, 4, 16, 2, 24, 2, 16, 8, 24, 2, 16, 1),
    # layer sizes near TinyLlama's (width 2048, feed-forward 5632)
    "zadurax-2048": _zadurax(2048, 32000, 5632, 32, 64, 4, 1024, 16, 64, 32, 256, 16, 128, 1),
    # ... and near Llama-2-7B's (width 4096, feed-forward 11008)
    "zadurax-4096": _zadurax(4096, 32000, 11008, 32, 128, 8, 1024, 32, 128, 64, 512, 16, 256, 1),
})


def _pudulorn(width, vocab, ff, heads, kv_heads, dim, vdim, chunk, latent_heads, latent_dim, rot_dim, kv_rank, q_rank,
              window, experts, top, expert_ff, blocks):
    """`blocks` times: differential attention with a dense feed-forward, latent attention with a mixture of experts,
    differential attention again, and a latent layer that reads the cached latent of the block's first one."""
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff, "limit": 7.0},
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": 0.8,
                           "mask": {"size": chunk}, "rot": {"base": 10000.0, "dims": dim}, "scale": dim ** -0.5}}
    latent = {"type": "latent_attention",
              "mlp": {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": 1.0},
                      "shared": {"ff": expert_ff}},
              "mixer": {"heads": latent_heads, "dim": latent_dim, "rot_dim": rot_dim, "vdim": latent_dim, "kv_rank": kv_rank,
                        "q_rank": q_rank, "mask": {"size": window}, "rot": {"base": 10000.0, "dims": rot_dim},
                        "scale": (latent_dim + rot_dim) ** -0.5}}
    layers = []
    for b in range(blocks):
        layers += [attention, latent, attention, dict(latent, mixer=dict(latent["mixer"], kv_from=4 * b + 1))]
    return dict(architecture="Pudulorn", vocab=vocab, width=width, norm={"eps": 1e-6}, layers=layers)


PRESETS.update({
    "pudulorn-tiny": _pudulorn(64, 300, 96, 4, 2, 16, 24, 24, 2, 16, 8, 24, 32, 20, 4, 2, 32, 1),
    # layer sizes near TinyLlama's (width 2048, feed-forward 5632): 16 heads of two maps of 64, values of 128;
    # eight experts of which two (plus the shared one) give a token 3 x 1,408 feed-forward rows of the dense 5,632 x 3/4
    "pudulorn-2048": _pudulorn(2048, 32000, 5632, 16, 4, 64, 128, 1024, 16, 64, 32, 256, 768, 1024, 8, 2, 1408, 2),
    # ... and near Llama-2-7B's (width 4096, feed-forward 11008)
    "pudulorn-4096": _pudulorn(4096, 32000, 11008, 16, 8, 128, 256, 1024, 32, 128, 64, 512, 1536, 1024, 8, 2, 2752, 2),
})


def _gurolix(width, vocab, blocks, heads, kv_heads, dim, vdim, state_heads, state_vdim, state, state_groups, experts, top,
             identity, groups, ff):
    """`blocks` times: capped attention, Mamba-2, normed attention, Mamba-2, each with a mixture of experts."""
    mlp = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "top": top, "identity": identity, "groups": {"count": groups[0], "keep": groups[1]}}}
    common = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "v_mix": True}
    capped = {"type": "attention_2", "mlp": mlp,
              "mixer": dict(common, softcap=30.0, rot={"base": 500000.0, "dims": dim, "scaling": {
                  "factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}})}
    normed = {"type": "attention", "mlp": mlp, "mixer": dict(common, rot={"base": 10000.0, "dims": dim // 2})}
    ssm = {"type": "mamba2", "mlp": mlp,
           "mixer": {"heads": state_heads, "vdim": state_vdim, "state": state, "groups": state_groups, "conv": 4,
                     "norm_groups": state_groups}}
    return dict(architecture="Gurolix", vocab=vocab, width=width, norm={"eps": 1e-5}, layers=[capped, ssm, normed, ssm] * blocks)


PRESETS.update({
    "gurolix-tiny": _gurolix(64, 300, 1, 4, 2, 16, 8, 4, 8, 16, 2, 5, 2, 1, (3, 2), 32),
    # widths and expert sizes of the Pudulorn presets; attention heads of 128 with values of 64 (of 128 at the larger
    # size), Mamba-2 with twice the width inside, heads of 64 and states of 128
    "gurolix-2048": _gurolix(2048, 32000, 1, 16, 4, 128, 64, 64, 64, 128, 8, 8, 2, 2, (5, 3), 1408),
    "gurolix-4096": _gurolix(4096, 32000, 1, 32, 8, 128, 128, 128, 64, 128, 8, 8, 2, 2, (5, 3), 2752),
})


def preset_config(name: str, **overrides):
    from ..config.llama import LlamaConfig
    from ..errors import ConfigError

    if name not in PRESETS:
        raise ConfigError(f"unknown preset '{name}' (known: {sorted(PRESETS)})")
    if "architecture" in PRESETS[name]:
        import copy
        from ..config.registry import resolve_architecture
        d = copy.deepcopy(PRESETS[name])
        d.update(overrides)
        return resolve_architecture(d).config_class.from_dict(d)
    d = dict(PRESETS[name], architectures=["LlamaForCausalLM"])
    d.update(overrides)
    return LlamaConfig.from_dict(d)
