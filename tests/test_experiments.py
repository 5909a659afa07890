"""The experiment scripts launch commands that this command line accepts.

Each script runs with a stand-in ``python`` on PATH that records its arguments instead of training;
what follows ``-m diloco_swarm_b200.train`` must parse into a Config with the topology, optimisers and
batch sizes of the reference's runs (experiments/experiment{1,2,3}.sh, experiments/test.sh)."""
import os
import stat
import subprocess

from diloco_swarm_b200.config import config_from_argv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def recorded_launches(script, tmp_path, env=None):
    fake = tmp_path / "bin"
    fake.mkdir()
    log = tmp_path / "calls.jsonl"
    py = fake / "python"
    py.write_text("#!/bin/bash\nprintf '%s\\n' \"$(printf '%s\\x1f' \"$@\")\" >> " + str(log) + "\n")
    py.chmod(py.stat().st_mode | stat.S_IEXEC)
    e = dict(os.environ, PATH=f"{fake}:{os.environ['PATH']}", DATA="@configs/data/synthetic-zipf.toml", **(env or {}))
    subprocess.run(["bash", os.path.join(ROOT, "experiments", script)], cwd=ROOT, env=e, check=True, timeout=60)
    calls = [line.rstrip("\n").split("\x1f")[:-1] for line in open(log)]
    out = []
    for argv in calls:
        if "diloco_swarm_b200.train" not in argv:
            continue                              # e.g. the table command at the end of benchmark.sh
        i = argv.index("diloco_swarm_b200.train")
        nproc = int(argv[argv.index("--nproc-per-node") + 1])
        out.append((nproc, config_from_argv(argv[i + 1:])))
    return out


def test_experiment1_launches(tmp_path):
    runs = recorded_launches("experiment1.sh", tmp_path)
    assert [(n, c.swarm.num_stages, c.swarm.sync_every_n_steps, c.train.outer_optimizer.type) for n, c in runs] == \
        [(1, 1, 1, "None"), (8, 2, 1, "None"), (8, 2, 50, "SGD")]
    single, swarm, diloco = (c for _, c in runs)
    assert (single.train.batch_size, single.train.micro_batch_size) == (512, 64)
    assert (swarm.train.batch_size, swarm.train.micro_batch_size, swarm.train.max_micro_batches) == (2048, 32, 12)
    assert diloco.train.outer_optimizer.nesterov and diloco.train.outer_optimizer.lr == 0.7
    assert all(c.model.n_layer == 12 and c.train.inner_optimizer.lr == 4e-4 and c.train.scheduler.num_warmup_steps == 50
               and c.train.max_steps == 2000 and c.data.seq_length == 1024 for _, c in runs)


def test_experiment2_sweeps_the_sync_interval(tmp_path):
    runs = recorded_launches("experiment2.sh", tmp_path, {"HS": "10 50 200"})
    assert [c.swarm.sync_every_n_steps for _, c in runs] == [10, 50, 200]
    assert [c.logging.run_id for _, c in runs] == ["diloco-H10", "diloco-H50", "diloco-H200"]
    assert all(n == 8 and c.train.outer_optimizer.type == "SGD" and c.eval.every_n_steps == c.swarm.sync_every_n_steps
               for n, c in runs)


def test_experiment3_sweeps_the_model_size(tmp_path):
    runs = recorded_launches("experiment3.sh", tmp_path, {"MEDIUM_STAGES": "4"})
    assert [(c.model.n_layer, c.model.n_embd, c.train.micro_batch_size, c.train.max_micro_batches, c.swarm.num_stages)
            for _, c in runs] == [(4, 128, 64, 16, 2), (24, 1024, 8, 16, 4), (36, 1280, 4, 8, 2)]
    assert all(c.swarm.layer_split == "balanced" and c.swarm.sync_every_n_steps == 50 for _, c in runs)


def test_smoke_script_launch(tmp_path):
    (n, c), = recorded_launches("test.sh", tmp_path)
    assert n == 2 and c.swarm.num_stages == 1 and c.device == "cpu" and c.data.tokenize and c.train.max_steps == 40


def test_benchmark_script_covers_the_four_kinds_of_parallelism(tmp_path):
    from diloco_swarm_b200.utils.results import parallelism
    runs = recorded_launches("benchmark.sh", tmp_path, {"GPUS": "4", "MBS": "16", "CAPS": "8", "OUT": str(tmp_path / "out")})
    kinds = [parallelism(n, c.swarm.num_stages) for n, c in runs]
    assert kinds == ["Single GPU", "Data Parallel", "Pipeline Parallel", "Pipeline Parallel", "SWARM"]
    assert [c.logging.run_id for _, c in runs] == ["single-mbs16", "dp4-mbs16", "pp2-mbs16-cap8", "pp4-mbs16-cap8",
                                                   "swarm4-mbs16-cap8"]
    assert all(c.train.batch_size == 512 and c.train.micro_batch_size == 16 and c.train.max_steps == 5 and
               c.model.n_embd == 768 and c.data.seq_length == 1024 for _, c in runs)
