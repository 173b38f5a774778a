"""Declarative table binding each rollout family to its collector settings,
executor, runtime builder, spec extractor and chunk gatherer
(reference: ``vrl/rollouts/families/specs.py:17-259``).  Everything is an import
path or a tuple of field names so the table can be read without importing models.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

CollectorKind = Literal["diffusion", "ar_discrete", "ar_continuous"]


@dataclass(frozen=True, slots=True)
class CollectorMetadata:
    kind: CollectorKind
    config_cls: str
    request_prefix: str | None = None
    default_task_type: str | None = None
    error_prefix: str | None = None
    sampling_fields: tuple[str, ...] = ()
    return_artifacts: tuple[str, ...] = ()
    metadata_key: str | None = None


@dataclass(frozen=True, slots=True)
class ExecutorKwargsMetadata:
    include_sample_batch_size: bool = False
    include_reference_image: bool = False


@dataclass(frozen=True, slots=True)
class GathererMetadata:
    import_path: str
    kwargs: dict[str, object] = field(default_factory=dict)


@dataclass(frozen=True, slots=True)
class RolloutFamilyEntry:
    family: str
    task: str
    collector: CollectorMetadata
    executor_cls: str
    runtime_builder: str
    runtime_spec_extractor: str
    gatherer: GathererMetadata
    executor_kwargs: ExecutorKwargsMetadata = field(default_factory=ExecutorKwargsMetadata)
    aliases: tuple[str, ...] = ()


DIFFUSION_RETURN_ARTIFACTS = ("output", "rollout_trajectory_data", "trajectory_timesteps",
                              "trajectory_latents", "denoising_env")
DIFFUSION_COMMON_SAMPLING_FIELDS = (
    "num_steps", "guidance_scale", "height", "width", "cfg", "sample_batch_size", "sde_type",
    "sde_window_size", "sde_window_range", "same_latent", "max_sequence_length", "noise_level",
    "return_kl",
)
DIFFUSION_VIDEO_SAMPLING_FIELDS = (*DIFFUSION_COMMON_SAMPLING_FIELDS, "num_frames")

_CFG = "visionrl_b200.rollouts.collector.configs"
_FAM = "visionrl_b200.models.families"
_DIFF_GATHER = "visionrl_b200.engine.gather:DiffusionChunkGatherer"


def _diffusion(family, task, aliases, cfg_cls, task_type, label, fields, module, stem,
               gather_kwargs=None, ref_image=False) -> RolloutFamilyEntry:
    return RolloutFamilyEntry(
        family=family, task=task, aliases=aliases,
        collector=CollectorMetadata(
            kind="diffusion", config_cls=f"{_CFG}:{cfg_cls}", request_prefix=family,
            default_task_type=task_type, error_prefix=label, sampling_fields=fields,
            return_artifacts=DIFFUSION_RETURN_ARTIFACTS),
        executor_cls=f"{_FAM}.{module}.executor:{stem[0]}",
        runtime_builder=f"{_FAM}.{module}.builder:build_{stem[1]}_runtime_bundle",
        runtime_spec_extractor=f"{_FAM}.{module}.builder:extract_{stem[1]}_runtime_spec",
        gatherer=GathererMetadata(_DIFF_GATHER, {"model_family": family, **(gather_kwargs or {})}),
        executor_kwargs=ExecutorKwargsMetadata(include_sample_batch_size=True,
                                               include_reference_image=ref_image),
    )


def _ar(family, aliases, kind, cfg_cls, fields, artifacts, module, stem,
        metadata_key=None) -> RolloutFamilyEntry:
    return RolloutFamilyEntry(
        family=family, task="ar_t2i", aliases=aliases,
        collector=CollectorMetadata(
            kind=kind, config_cls=f"{_CFG}:{cfg_cls}", request_prefix=family,
            sampling_fields=fields, return_artifacts=artifacts, metadata_key=metadata_key),
        executor_cls=f"{_FAM}.{module}.executor:{stem[0]}PipelineExecutor",
        runtime_builder=f"{_FAM}.{module}.builder:build_{module}_runtime_bundle",
        runtime_spec_extractor=f"{_FAM}.{module}.builder:extract_{module}_runtime_spec",
        gatherer=GathererMetadata(f"{_FAM}.{module}.executor:{stem[0]}ChunkGatherer"),
    )


FAMILY_REGISTRY: dict[str, RolloutFamilyEntry] = {
    "sd3_5": _diffusion("sd3_5", "t2i", ("sd3.5", "sd35"), "SD3_5CollectorConfig",
                        "text_to_image", "SD3.5", DIFFUSION_COMMON_SAMPLING_FIELDS, "sd3_5",
                        ("SD3_5PipelineExecutor", "sd3_5")),
    "wan_2_1": _diffusion("wan_2_1", "t2v", ("wan", "wan_2_1_1_3b", "wan_2_1_14b"),
                          "Wan_2_1CollectorConfig", "text_to_video", "Wan 2.1",
                          DIFFUSION_VIDEO_SAMPLING_FIELDS, "wan_2_1",
                          ("Wan_2_1PipelineExecutor", "wan_2_1")),
    "cosmos": _diffusion("cosmos", "v2w", ("cosmos_predict2", "cosmos_predict2_2b"),
                         "CosmosPredict2CollectorConfig", "video2world", "Cosmos",
                         (*DIFFUSION_VIDEO_SAMPLING_FIELDS, "fps"), "cosmos",
                         ("CosmosPipelineExecutor", "cosmos_predict2"),
                         gather_kwargs={"respect_cfg_flag": False}, ref_image=True),
    "janus_pro": _ar("janus_pro", ("janus", "janus_pro_1b"), "ar_discrete",
                     "JanusProCollectorConfig",
                     ("cfg_weight", "temperature", "image_token_num", "image_size",
                      "max_text_length"),
                     ("output", "token_ids", "token_log_probs"), "janus_pro", ("JanusPro",)),
    "nextstep_1": _ar("nextstep_1", ("nextstep", "nextstep_1_1"), "ar_continuous",
                      "NextStep1CollectorConfig",
                      ("cfg_scale", "num_flow_steps", "noise_level", "image_token_num",
                       "image_size", "max_text_length", "rescale_to_unit"),
                      ("output", "rollout_trajectory_data"), "nextstep_1", ("NextStep1",),
                      metadata_key="rollout_metadata"),
}

_ALIASES = {alias: fam for fam, e in FAMILY_REGISTRY.items() for alias in (fam, *e.aliases)}


def normalize_rollout_family(family: str) -> str:
    return _ALIASES.get(str(family), str(family))


def get_rollout_family_entry(family: str) -> RolloutFamilyEntry:
    key = normalize_rollout_family(family)
    if key not in FAMILY_REGISTRY:
        raise ValueError(
            f"unsupported rollout family: {family!r}; registered={sorted(FAMILY_REGISTRY)}")
    return FAMILY_REGISTRY[key]


def registered_rollout_families() -> tuple[str, ...]:
    return tuple(FAMILY_REGISTRY)


__all__ = [
    "DIFFUSION_COMMON_SAMPLING_FIELDS", "DIFFUSION_RETURN_ARTIFACTS",
    "DIFFUSION_VIDEO_SAMPLING_FIELDS", "FAMILY_REGISTRY", "CollectorKind", "CollectorMetadata",
    "ExecutorKwargsMetadata", "GathererMetadata", "RolloutFamilyEntry",
    "get_rollout_family_entry", "normalize_rollout_family", "registered_rollout_families",
]
