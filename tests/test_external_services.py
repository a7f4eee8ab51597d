# SPDX-License-Identifier: Apache-2.0
"""Launchers and data sources that talk to external services, exercised against fakes (no Ray, no Snowflake installed).

Pattern of the reference's mocked Snowflake tests (tests/data/test_snowflake_source.py:28-372): configuration rules,
and the load paths with the client library replaced by stand-ins that record how they were called."""

import sys
import types
from pathlib import Path

import pytest
import yaml

ROOT = Path(__file__).resolve().parent.parent


# ----------------------------------------------------------------------------------------------- Snowflake
@pytest.fixture
def fake_snowflake(monkeypatch):
    calls = {}

    class FakeConnector:
        def __init__(self, kind, arg):
            self.kind, self.arg = kind, arg

        @classmethod
        def from_sql(cls, sql, session=None):
            calls["from_sql"] = (sql, session)
            return cls("sql", sql)

        @classmethod
        def from_dataset(cls, ds):
            calls["from_dataset"] = ds
            return cls("dataset", ds)

        def to_huggingface_dataset(self, streaming=False, limit=None, batch_size=1024):
            import datasets

            calls["to_hf"] = dict(streaming=streaming, limit=limit, batch_size=batch_size)
            rows = [{"TXT": f"row {i}", "N": i} for i in range(6)]
            return datasets.Dataset.from_list(rows[: limit or len(rows)])

    def load_dataset(session, name, version):
        calls["load_dataset"] = (session, name, version)
        return ("dataset-object", name, version)

    mods = {
        "snowflake": types.ModuleType("snowflake"),
        "snowflake.ml": types.ModuleType("snowflake.ml"),
        "snowflake.ml.data": types.ModuleType("snowflake.ml.data"),
        "snowflake.ml.data.data_connector": types.ModuleType("snowflake.ml.data.data_connector"),
        "snowflake.ml.dataset": types.ModuleType("snowflake.ml.dataset"),
    }
    mods["snowflake.ml.data.data_connector"].DataConnector = FakeConnector
    mods["snowflake.ml.dataset"].load_dataset = load_dataset
    for name, mod in mods.items():
        monkeypatch.setitem(sys.modules, name, mod)
    return calls


def _source(cfg_kwargs, session="SESSION"):
    from types import SimpleNamespace

    from arctictraining_b200.data.snowflake import SnowflakeDataSource
    from arctictraining_b200.data.snowflake import SnowflakeSourceConfig

    cfg = SnowflakeSourceConfig(type="snowflake", **cfg_kwargs)
    src = SnowflakeDataSource.__new__(SnowflakeDataSource)
    src.config = cfg
    src.session = session
    src._data_factory = SimpleNamespace()
    return src, cfg


def test_snowflake_modes_are_mutually_exclusive_and_uris_are_validated():
    from arctictraining_b200.data.snowflake import SnowflakeSourceConfig

    with pytest.raises(ValueError, match="Exactly one"):
        SnowflakeSourceConfig(type="snowflake")
    with pytest.raises(ValueError, match="Exactly one"):
        SnowflakeSourceConfig(type="snowflake", sql="select 1", table_name="T")
    with pytest.raises(ValueError, match="Invalid dataset_uri"):
        SnowflakeSourceConfig(type="snowflake", dataset_uri="snow://wrong/ds/versions/v1")
    with pytest.raises(ValueError, match="Invalid dataset_name"):
        SnowflakeSourceConfig(type="snowflake", dataset_uri="snow://dataset/bad name/versions/v1")
    ok = SnowflakeSourceConfig(type="snowflake", table_name="DB.SCHEMA.T")
    assert ok.sql == "SELECT * FROM DB.SCHEMA.T"


def test_snowflake_sql_load_passes_the_session_limit_and_batch_size(fake_snowflake):
    src, cfg = _source({"sql": "SELECT TXT, N FROM T", "limit": 4, "batch_size": 77, "column_mapping": {"TXT": "text"}})
    ds = src.load(cfg, "train")
    assert fake_snowflake["from_sql"] == ("SELECT TXT, N FROM T", "SESSION")
    assert fake_snowflake["to_hf"] == {"streaming": False, "limit": 4, "batch_size": 77}
    assert len(ds) == 4
    # the renaming runs as the source's post-load callback
    assert "text" in ds.column_names and "TXT" not in ds.column_names


def test_snowflake_dataset_uri_load_resolves_name_and_version(fake_snowflake):
    src, cfg = _source({"dataset_uri": "snow://dataset/DB.SCH.MYDS/versions/v3"})
    ds = src.load(cfg, "train")
    assert fake_snowflake["load_dataset"] == ("SESSION", "DB.SCH.MYDS", "v3")
    assert fake_snowflake["from_dataset"] == ("dataset-object", "DB.SCH.MYDS", "v3")
    assert "from_sql" not in fake_snowflake and len(ds) == 6


def test_snowflake_load_without_the_client_library_says_what_is_missing(monkeypatch):
    for name in [m for m in sys.modules if m == "snowflake" or m.startswith("snowflake.")]:
        monkeypatch.delitem(sys.modules, name)
    monkeypatch.setitem(sys.modules, "snowflake", None)
    src, cfg = _source({"sql": "select 1"})
    with pytest.raises(ImportError, match="snowflake-ml-python"):
        src.load(cfg, "train")


# ----------------------------------------------------------------------------------------------- Ray
@pytest.fixture
def fake_ray(monkeypatch):
    """A stand-in for ``ray`` / ``ray.train``: ``TorchTrainer.fit`` runs the per-worker loop once in this process."""
    rec = {"reports": [], "init": 0}
    ray = types.ModuleType("ray")
    train = types.ModuleType("ray.train")
    train_torch = types.ModuleType("ray.train.torch")
    ray.is_initialized = lambda: False
    ray.init = lambda *a, **k: rec.__setitem__("init", rec["init"] + 1)
    ray.cluster_resources = lambda: {"GPU": 0, "CPU": 4}

    class ScalingConfig:
        def __init__(self, num_workers, use_gpu):
            rec["scaling"] = (num_workers, use_gpu)

    class RunConfig:
        def __init__(self, storage_path=None):
            rec["storage_path"] = storage_path

    class Checkpoint:
        @classmethod
        def from_directory(cls, d):
            rec["checkpoint_dir"] = d
            return ("ckpt", d)

    class _Ctx:
        def get_storage(self):
            return types.SimpleNamespace(storage_fs_path=rec.get("storage_root", "/nonexistent-storage-root"))

    train.ScalingConfig, train.RunConfig, train.Checkpoint = ScalingConfig, RunConfig, Checkpoint
    train.get_context = lambda: _Ctx()
    train.report = lambda metrics, **kw: rec["reports"].append((dict(metrics), kw))

    class TorchTrainer:
        def __init__(self, loop, train_loop_config, scaling_config, run_config):
            self.loop, self.cfg = loop, train_loop_config

        def fit(self):
            self.loop(self.cfg)
            return "fit-result"

    train_torch.TorchTrainer = TorchTrainer
    ray.train = train
    train.torch = train_torch
    for name, mod in {"ray": ray, "ray.train": train, "ray.train.torch": train_torch}.items():
        monkeypatch.setitem(sys.modules, name, mod)
    return rec


def test_ray_launcher_runs_the_trainer_and_reports_metrics_and_checkpoints(fake_ray, tiny_recipe, tmp_path):
    from arctictraining_b200.launcher import ray_launcher

    recipe = tiny_recipe(exit_iteration=3, train_log_iter_interval=1,
                         checkpoint=[{"type": "huggingface", "output_dir": str(tmp_path / "hf"), "save_end_of_training": True}])
    path = tmp_path / "recipe.yaml"
    path.write_text(yaml.safe_dump(recipe))
    out = ray_launcher.launch(str(path), num_workers=None)
    assert out == "fit-result" and fake_ray["init"] == 1
    assert fake_ray["scaling"] == (1, False)          # no GPU in the fake cluster: one CPU worker
    step_reports = [m for m, kw in fake_ray["reports"] if "checkpoint" not in kw]
    assert len(step_reports) == 2 and all("loss" in m for m in step_reports)  # iterations 1 and 2; 3 goes with the checkpoint
    ckpt_reports = [kw for m, kw in fake_ray["reports"] if kw.get("checkpoint")]
    assert ckpt_reports and fake_ray["checkpoint_dir"].endswith("global_step_3")


def test_ray_launcher_moves_relative_outputs_under_the_job_stage(monkeypatch):
    from arctictraining_b200.launcher.ray_launcher import stage_paths_from_env

    cfg = {"checkpoint": [{"output_dir": "ckpts/run1"}, {"output_dir": "/abs/elsewhere"}]}
    assert stage_paths_from_env({"checkpoint": [{"output_dir": "x"}]})["checkpoint"][0]["output_dir"] == "x"
    monkeypatch.setenv("MLRS_STAGE_MOUNT_PATH", "/mnt/stage")
    monkeypatch.setenv("MLRS_STAGE_RESULT_PATH", "results")
    out = stage_paths_from_env(cfg)
    assert out["checkpoint"][0]["output_dir"] == "/mnt/stage/results/ckpts/run1"
    assert out["checkpoint"][1]["output_dir"] == "/abs/elsewhere"


def test_wandb_run_receives_config_metrics_and_finish(tiny_recipe, monkeypatch, tmp_path):
    """Weights & Biases logging against a fake ``wandb`` module: one run is opened with the recipe as its config, the
    step metrics arrive with the step number, the run is finished, and its id survives in the checkpoint state so that
    a resumed job continues the same run (the reference keeps this in arctic_training/trainer/trainer.py:305-330)."""
    import sys
    import types

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    calls = {"init": [], "log": [], "finish": 0}

    class Run:
        def log(self, data, step=None):
            calls["log"].append((dict(data), step))

        def finish(self):
            calls["finish"] += 1

    fake = types.ModuleType("wandb")
    fake.util = types.SimpleNamespace(generate_id=lambda: "run123")
    fake.init = lambda **kw: (calls["init"].append(kw), Run())[1]
    monkeypatch.setitem(sys.modules, "wandb", fake)

    import yaml

    r = tiny_recipe(exit_iteration=4, train_log_iter_interval=1, wandb={"enable": True, "project": "proj", "name": "unit"})
    p = tmp_path / "wandb.yaml"
    p.write_text(yaml.safe_dump(r))
    cfg = get_config(p)
    tr = get_registered_trainer(cfg.type)(cfg)
    tr.train()
    assert len(calls["init"]) == 1
    init = calls["init"][0]
    assert init["project"] == "proj" and init["name"] == "unit" and init["id"] == "run123" and init["resume"] == "allow"
    assert init["config"]["type"] == "sft" and init["config"]["model"]["name_or_path"] == "tiny-llama"
    steps = [s for _, s in calls["log"]]
    assert steps and steps == sorted(steps) and all("loss" in d for d, _ in calls["log"])
    assert calls["finish"] == 1
    assert tr.wandb_run_id == "run123"
