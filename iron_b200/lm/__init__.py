"""Language-model layer: configs, blocks, the causal graph, the fused engine, checkpoints, the CLI."""


#: the names ``iron.lm`` exports (iron/lm/__init__.py:46-94) that this library holds, by module
_EXPORTS = {
    "blocks": ("Attention", "Call", "DecoderLayer", "Embedding", "GatedMLP", "KVCache", "Linear", "RMSNorm", "Rope",
               "residual_add"),
    "causal": ("CausalConv1d", "CausalLM", "Checkpoints", "Decoder"),
    "config": ("Config", "DecoderConfig", "Precision", "not_json", "rope_angles"),
    "generation": ("Sampler", "generate_on_host", "greedy"),
    "engine": ("LlamaEngine",),
    "mamba": ("MambaMixer",),
}


def __getattr__(name):
    # ``from iron_b200.lm import Checkpoint`` as ``iron.lm`` exports it, without importing
    # torch for code that only reads configs
    if name in ("Checkpoint", "weights_file", "leaves", "nest", "subtree", "renamed", "save_file", "Uploader"):
        from . import checkpoint

        return getattr(checkpoint, name)
    if name == "main":
        from .cli import main

        return main
    for module, names in _EXPORTS.items():
        if name in names:
            import importlib

            return getattr(importlib.import_module(f"{__name__}.{module}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
