"""`python -m sglang_jax_b200.launch_server --model-path ... [--tp 8 ...]`
(reference `python/sgl_jax/launch_server.py:10-31`)."""

import sys

from .server_args import prepare_server_args


def main(argv=None):
    server_args = prepare_server_args(argv if argv is not None else sys.argv[1:])
    if server_args.multimodal:
        from .multimodal.entrypoint.http_server import launch as launch_mm
        launch_mm(server_args)
        return
    from .entrypoints.http_server import launch
    launch(server_args)


if __name__ == "__main__":
    main()
