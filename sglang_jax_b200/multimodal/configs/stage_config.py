"""Stage pipeline description loaded from YAML (reference `multimodal/models/static_configs/*.yaml`,
`multimodal/configs/config_registry.py`)."""

from __future__ import annotations

import dataclasses
import os

import yaml

STATIC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "models", "static_configs")


@dataclasses.dataclass
class StageConfig:
    stage_id: int
    scheduler: str                      # text_encoder | diffusion | vae | vit | embed | audio_encoder | audio_backbone | llm
    model_class: str
    stage_sub_dir: str = ""
    num_gpus: int = 1
    max_batch_size: int = 1
    final_output: bool = False
    scheduler_params: dict = dataclasses.field(default_factory=dict)
    model_path: str | None = None


@dataclasses.dataclass
class PipelineConfig:
    model_arch: str
    stages: list[StageConfig]

    @classmethod
    def from_yaml(cls, path: str) -> "PipelineConfig":
        with open(path) as f:
            d = yaml.safe_load(f)
        stages = []
        for s in d["stage_args"]:
            rt = s.get("runtime", {}) or {}
            stages.append(StageConfig(
                stage_id=int(s["stage_id"]), scheduler=s["scheduler"], model_class=s["model_class"],
                stage_sub_dir=s.get("stage_sub_dir", ""), num_gpus=int(rt.get("num_gpus", rt.get("num_tpus", 1))),
                max_batch_size=int(rt.get("max_batch_size", 1)), final_output=bool(s.get("final_output", False)),
                scheduler_params=s.get("scheduler_params") or {}, model_path=s.get("model_path")))
        stages.sort(key=lambda x: x.stage_id)
        if not stages or not stages[-1].final_output:
            raise ValueError(f"{path}: the last stage must set final_output")
        return cls(d["model_arch"], stages)


def registry() -> dict[str, str]:
    """model_arch -> YAML path for every bundled pipeline."""
    out = {}
    for f in sorted(os.listdir(STATIC_DIR)):
        if f.endswith(".yaml"):
            with open(os.path.join(STATIC_DIR, f)) as fh:
                out[yaml.safe_load(fh)["model_arch"]] = os.path.join(STATIC_DIR, f)
    return out


def resolve(model_arch_or_path: str) -> PipelineConfig:
    if os.path.isfile(model_arch_or_path):
        return PipelineConfig.from_yaml(model_arch_or_path)
    reg = registry()
    for arch, path in reg.items():
        if arch == model_arch_or_path or arch.split("/")[-1].lower() in model_arch_or_path.lower():
            return PipelineConfig.from_yaml(path)
    raise ValueError(f"no stage config for {model_arch_or_path!r}; known: {sorted(reg)}")
