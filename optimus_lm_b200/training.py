"""``ParallelTrainer`` for pipeline parallelism with GPipe and non-interleaved 1F1B - the trainer
the driver uses by default when PP > 1.  Same constructor and ``step`` signature as the
reference's optimus/training.py:18-497; the work is done by ``pipeline.PipelineExecutor``."""
from .pipeline import ParallelTrainerOutput, PipelineExecutor  # noqa: F401


class ParallelTrainer(PipelineExecutor):
    def __init__(self, config, model, pmap, batch_size, micro_batch_size, context_size, opt_grad_acc_steps, dtype,
                 device, pp_scheme="gpipe", reuse_buffers_in_1f1b=True, verbose=False, memory_tracker=None):
        assert getattr(config, "virtual_pipeline_parallelism", 1) == 1, \
            "virtual pipeline parallelism needs optimus_lm_b200.trainer.ParallelTrainer (--use_latest_trainer)"
        super().__init__(config, model, pmap, batch_size, micro_batch_size, context_size, opt_grad_acc_steps, dtype,
                         device, pp_scheme=pp_scheme, reuse_buffers_in_1f1b=reuse_buffers_in_1f1b, verbose=verbose,
                         memory_tracker=memory_tracker)
