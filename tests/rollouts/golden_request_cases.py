"""What each family's collector asks the engine for: the collector configuration defaults of the
five families and the generation request built for a plain and for a fully specified ``collect``
call (family, task, prompts, group size, the sampling dictionary, metadata, policy version,
requested artifacts, the shape of the request id).  ``compute()`` returns them as JSON strings;
``tests/golden/collector_requests.json`` holds what the reference's collectors build."""

import asyncio
import dataclasses
import json

from vrl.engine.core.types import OutputBatch, GenerationMetrics
from vrl.rollouts.collector import (build_rollout_collector, SD3_5CollectorConfig, Wan_2_1CollectorConfig, CosmosPredict2CollectorConfig,
                                    JanusProCollectorConfig, NextStep1CollectorConfig)
import json


def compute() -> dict:
    res = {}
    class Runtime:
        def __init__(self): self.requests = []
        async def generate(self, request):
            self.requests.append(request)
            raise RuntimeError("stop after the request is built")
    loop = asyncio.new_event_loop()
    def norm(v):
        if isinstance(v, (set, frozenset)): return sorted(v)
        if isinstance(v, tuple): return list(v)
        return v
    for fam, cfg in (("sd3_5", SD3_5CollectorConfig()), ("wan_2_1", Wan_2_1CollectorConfig()), ("cosmos", CosmosPredict2CollectorConfig()),
                     ("janus_pro", JanusProCollectorConfig()), ("nextstep_1", NextStep1CollectorConfig())):
        res[f"{fam}/config"] = json.dumps({k: norm(v) for k, v in dataclasses.asdict(cfg).items()}, sort_keys=True, default=str)
        rt = Runtime()
        col = build_rollout_collector(fam, model=None, reward_fn=None, config=cfg, runtime=rt)
        for label, kw in (("plain", {}), ("rich", {"seed": 7, "target_text": "HELLO", "references": ["r"], "task_type": "ocr", "sample_metadata": {"k": 1},
                                                   "request_overrides": {"guidance_scale": 2.0}, "policy_version": 5})):
            try: loop.run_until_complete(col.collect(["a prompt", "b"], group_size=3, **kw))
            except Exception as e: pass
            r = rt.requests[-1]
            d = {"family": r.family, "task": r.task, "prompts": list(r.prompts), "n": r.samples_per_prompt, "sampling": {k: norm(v) for k, v in sorted(r.sampling.items())},
                 "metadata": r.metadata, "policy_version": r.policy_version, "return_artifacts": norm(r.return_artifacts), "id_prefix": r.request_id.split("-", 1)[0], "id_parts": len(r.request_id.split("-"))}
            res[f"{fam}/{label}"] = json.dumps(d, sort_keys=True, default=str)
    return res
