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

import os as _os

# CUDA loads kernels lazily by default, and the first launch of a kernel can wait
# for everything running on the device.  With a pipeline receive already spinning
# on the GPU for a peer that is itself waiting for this rank, that wait never ends.
# Loading every module when the context is created removes the hazard (this has to
# be set before CUDA is initialised, hence at import).
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
