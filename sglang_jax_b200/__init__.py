"""B200-native LLM serving framework with the capabilities and public API of SGL-JAX.

    from sglang_jax_b200 import Engine
    engine = Engine(model_path=..., tp_size=8)
    engine.generate(prompt="...", sampling_params={"max_new_tokens": 32})

    python -m sglang_jax_b200.launch_server --model-path ... --tp 8
"""

__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .entrypoints.engine import Engine
        return Engine
    if name == "ServerArgs":
        from .server_args import ServerArgs
        return ServerArgs
    raise AttributeError(name)
