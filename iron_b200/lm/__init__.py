"""Language-model layer: configs, blocks, the causal graph, the fused engine, checkpoints, the CLI."""


def __getattr__(name):
    # ``from iron_b200.lm import Checkpoint`` as ``iron.lm`` exports it, without importing
    # torch for code that only reads configs
    if name in ("Checkpoint", "weights_file", "leaves", "nest", "subtree", "renamed", "save_file", "Uploader"):
        from . import checkpoint

        return getattr(checkpoint, name)
    if name == "main":
        from .cli import main

        return main
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
