# SPDX-License-Identifier: Apache-2.0
"""Ray Train launcher.  Behaviour parity: arctic_training/launcher/ray_launcher.py:40-209 — one Ray worker per GPU
(``TorchTrainer`` + ``ScalingConfig``), per-instance ``post-step`` (metrics report) and ``post-checkpoint`` (upload the
checkpoint directory) callbacks, Snowflake ML-job stage paths from ``MLRS_STAGE_MOUNT_PATH`` /
``MLRS_STAGE_RESULT_PATH``, optional cProfile on local rank 0.  Ray is imported lazily: the module loads without it.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Any
from typing import Dict
from typing import Optional

from ..callback.callback import Callback
from ..logging import logger


def _ray():
    try:
        import ray
        import ray.train
        import ray.train.torch  # noqa: F401
    except ImportError as exc:
        raise ImportError("the Ray launcher needs `ray[train]` (pip install 'ray[train]')") from exc
    return ray


def _post_step_ray_report(trainer) -> None:
    every = trainer.config.train_log_iter_interval
    # the summary of an iteration is assembled after its step: what is reported here is the previous iteration's
    # (nothing yet after the very first step)
    if trainer.gas_boundary and every and trainer.global_step % every == 0 and trainer.metrics.summary_dict:
        _ray().train.report(dict(trainer.metrics.summary_dict))


def _post_checkpoint_ray_save(trainer) -> None:
    ray = _ray()
    try:
        storage_root = Path(ray.train.get_context().get_storage().storage_fs_path).resolve()
    except AttributeError:
        logger.warning("Ray Train storage API not available: checkpoints are not uploaded to Ray Train.")
        return
    active = [e for e in trainer.checkpoint_engines if e.do_checkpoint]
    if not active:
        return
    kwargs: Dict[str, Any] = {"checkpoint": None}
    if trainer.global_rank == 0:
        inside = [e for e in active if e.checkpoint_dir.resolve().is_relative_to(storage_root)]
        if inside:
            try:
                from ray.train import CheckpointUploadMode

                kwargs["checkpoint"] = ray.train.Checkpoint.from_directory(inside[0].checkpoint_dir.as_posix())
                kwargs["checkpoint_upload_mode"] = CheckpointUploadMode.NO_UPLOAD
            except ImportError:
                pass
        else:
            kwargs["checkpoint"] = ray.train.Checkpoint.from_directory(active[0].checkpoint_dir.as_posix())
    ray.train.report(dict(trainer.metrics.summary_dict), **kwargs)


def attach_ray_callbacks(trainer) -> None:
    """Add the reporting callbacks to this trainer *instance* (other trainers of the class are unaffected)."""
    cls = type(trainer)
    methods = cls._get_all_callback_event_methods()
    extra = [Callback("post-step", _post_step_ray_report, methods["post-step"]),
             Callback("post-checkpoint", _post_checkpoint_ray_save, methods["post-checkpoint"])]
    trainer._initialized_callbacks = list(trainer._initialized_callbacks) + extra


def stage_paths_from_env(config_dict: Dict[str, Any]) -> Dict[str, Any]:
    """Inside a Snowflake ML job, relative output paths move under the mounted stage."""
    mount = os.getenv("MLRS_STAGE_MOUNT_PATH")
    result = os.getenv("MLRS_STAGE_RESULT_PATH")
    if not mount:
        return config_dict
    base = Path(mount) / (result or "")
    for ck in config_dict.get("checkpoint", []) or []:
        if "output_dir" in ck and not Path(ck["output_dir"]).is_absolute():
            ck["output_dir"] = str(base / ck["output_dir"])
    return config_dict


def _train_loop_per_worker(loop_config: Dict[str, Any]) -> None:
    from ..config.trainer import get_config
    from ..registry import get_registered_trainer

    config = get_config(Path(loop_config["config_file"]))
    trainer = get_registered_trainer(config.type)(config, mode=loop_config["mode"])
    attach_ray_callbacks(trainer)
    if loop_config["mode"] != "train":
        return
    profile = loop_config.get("python_profile", "disable")
    if profile == "disable" or config.local_rank != 0:
        trainer.train()
    else:
        import cProfile
        from pstats import SortKey

        cProfile.runctx("trainer.train()", None, {"trainer": trainer},
                        sort=SortKey.TIME if profile == "tottime" else SortKey.CUMULATIVE)


def launch(config_file: str, mode: str = "train", python_profile: str = "disable", num_workers: Optional[int] = None):
    ray = _ray()
    from ray.train import RunConfig
    from ray.train import ScalingConfig
    from ray.train.torch import TorchTrainer

    if not ray.is_initialized():
        ray.init()
    if num_workers is None:
        num_workers = int(ray.cluster_resources().get("GPU", 0)) or 1
    scaling = ScalingConfig(num_workers=num_workers, use_gpu=ray.cluster_resources().get("GPU", 0) > 0)
    storage = os.getenv("MLRS_STAGE_MOUNT_PATH")
    run_cfg = RunConfig(storage_path=storage) if storage else RunConfig()
    trainer = TorchTrainer(
        _train_loop_per_worker,
        train_loop_config={"config_file": str(Path(config_file).resolve()), "mode": mode, "python_profile": python_profile},
        scaling_config=scaling, run_config=run_cfg,
    )
    return trainer.fit()
