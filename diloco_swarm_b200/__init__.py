"""B200-native DiLoCo-SWARM training framework.

Layout:
  config      CLI grammar + schema
  world       S stages x R replicas topology and process groups
  models/     GPT-2 (autograd oracle) and the flat-buffer sm_100a stage
  ops/        Python entry points of the CUDA kernels (csrc/)
  parallel/   routing schedule, pipeline p2p, fused collectives, simulator
  utils/      logger, metrics, checkpoint, data, timers
  train       entry point (``python -m diloco_swarm_b200.train``)
"""
__version__ = "0.1.0"
