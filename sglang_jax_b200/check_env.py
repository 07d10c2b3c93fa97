"""`python -m sglang_jax_b200.check_env`: versions and hardware the framework sees."""

import importlib
import json
import platform


def check_env() -> dict:
    info = {"python": platform.python_version(), "platform": platform.platform()}
    for m in ("torch", "numpy", "transformers", "safetensors", "fastapi", "uvicorn", "zmq", "llguidance", "aiohttp"):
        try:
            info[m] = getattr(importlib.import_module(m), "__version__", "?")
        except Exception as e:
            info[m] = f"missing ({type(e).__name__})"
    try:
        import torch
        info["cuda_available"] = torch.cuda.is_available()
        if torch.cuda.is_available():
            info["gpus"] = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
            info["cuda"] = torch.version.cuda
            info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
        from .ops import native
        info["native_kernels"] = native.lib().sglb_version().decode()
    except Exception as e:
        info["native_kernels"] = f"unavailable ({e})"
    return info


if __name__ == "__main__":
    print(json.dumps(check_env(), indent=1))
