import os
from diloco_swarm_b200.config import Config


def make_config(**over) -> Config:
    base = {
        "model": {"n_layer": 2, "n_head": 4, "n_embd": 128, "vocab_size": 512, "block_size": 128},
        "data": {"path": "synthetic:zipf", "seq_length": 64, "num_examples": 64, "vocab_limit": 500},
        "train": {"micro_batch_size": 4, "batch_size": 16, "max_steps": 4, "max_micro_batches": 2,
                  "inner_optimizer": {"type": "AdamW", "lr": 1e-3},
                  "outer_optimizer": {"type": "None", "lr": 0.0}},
        "swarm": {"num_stages": 1},
        "amp": {"enable": False},
        "eval": {"enable": False}, "sample": {"enable": False},
        "logging": {"log_dir": "/tmp/dsw_tests", "console": {"log_level": "ERROR"}},
    }

    def upd(d, o):
        for k, v in o.items():
            if isinstance(v, dict) and isinstance(d.get(k), dict):
                upd(d[k], v)
            else:
                d[k] = v
    upd(base, over)
    return Config(**base)


def single_world(num_stages=1):
    from diloco_swarm_b200.world import World
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE"):
        os.environ.pop(k, None)
    return World(num_stages, init=False)
