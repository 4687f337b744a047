"""Asynchronous RL trainer: a generator loop and a trainer loop run concurrently in the controller, joined by a bounded
rollout queue (off-policy depth = ``--train.async_queue_size``) and a token pool that gives the generator
back-pressure; weight sync takes the engine lock (and optionally pauses generation for partial rollout).

Same protocol as openrlhf/trainer/ppo_trainer_async.py:19-353, with controller threads and the runtime's futures in
place of Ray actors and ``ray.util.queue``.
"""
from __future__ import annotations

import logging
import queue
import threading
import time

from ..runtime.core import get
from .ppo_trainer import PPOTrainer, compute_eval_metrics

logger = logging.getLogger(__name__)
DONE = "done"


class PPOTrainerAsync(PPOTrainer):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        q = max(1, self.args.train.async_queue_size)
        self.rollout_queue: queue.Queue = queue.Queue(maxsize=q)
        self.rollout_slots: queue.Queue = queue.Queue(maxsize=q)
        for _ in range(q):
            self.rollout_slots.put(0)
        self.engine_lock = threading.Lock()
        self.partial = self.args.train.partial_rollout_enable
        self._errors: list[BaseException] = []

    # ------------------------------------------------------------------ producer
    def _generator_loop(self, start_episode: int, consumed: int):
        a = self.args
        try:
            eval_just_done = False
            for episode in range(start_episode, a.train.num_episodes):
                self.samples_generator.restart_epoch()
                while True:
                    step_token = self.rollout_slots.get()          # blocks: back-pressure from the trainer
                    if (a.eval.steps > 0 and step_token and step_token % a.eval.steps == 0 and self.eval_dataloader
                            and not eval_just_done):
                        with self.engine_lock:
                            kw = dict(self.generate_kwargs, temperature=a.eval.temperature,
                                      n_samples_per_prompt=a.eval.n_samples_per_prompt)
                            ev = self.samples_generator.generate_eval_samples(**kw)
                        self.rollout_queue.put(("eval", step_token,
                                                compute_eval_metrics(self.eval_dataloader, ev, kw["n_samples_per_prompt"])))
                        eval_just_done = True
                    t0 = time.time()
                    if self.partial:
                        out = self.samples_generator.generate_samples(**self.generate_kwargs)
                    else:
                        with self.engine_lock:
                            out = self.samples_generator.generate_samples(**self.generate_kwargs)
                    samples, pass_rate, n_prompts, exhausted = out
                    consumed += n_prompts
                    if samples:
                        eval_just_done = False
                        dl = self.prompts_dataloader.state_dict() if hasattr(self.prompts_dataloader, "state_dict") else {}
                        self.rollout_queue.put((samples, {"episode": episode, "total_consumed_prompts": consumed,
                                                          "data_loader_state_dict": dl}, pass_rate, time.time() - t0))
                    else:
                        self.rollout_slots.put(step_token)         # nothing produced: hand the slot back
                    if exhausted:
                        break
        except BaseException as e:  # noqa: BLE001
            self._errors.append(e)
        finally:
            self.rollout_queue.put(DONE)

    # ------------------------------------------------------------------ consumer
    def broadcast_to_vllm(self):
        with self.engine_lock:
            if self.partial:
                get((self.groups.rollout or self.group).async_run_method("pause_generation"))
            try:
                super().broadcast_to_vllm()
            finally:
                if self.partial:
                    get((self.groups.rollout or self.group).async_run_method("resume_generation"))

    def fit(self, global_step: int = 0) -> None:
        a = self.args
        st = self.init_checkpoint_states()
        self.restore_best_checkpoint_state(st)
        if st["global_step"] > 0:
            global_step = st["global_step"]
            self.broadcast_to_vllm()
            if st.get("data_loader_state_dict") and hasattr(self.prompts_dataloader, "load_state_dict"):
                self.prompts_dataloader.load_state_dict(st["data_loader_state_dict"])
        producer = threading.Thread(target=self._generator_loop, args=(st["episode"], st["total_consumed_prompts"]),
                                    daemon=True)
        producer.start()
        last_cs = {}
        while True:
            t_wait = time.time()
            item = self.rollout_queue.get()
            if item == DONE:
                break
            if isinstance(item, tuple) and item[0] == "eval":
                _, step, logs = item
                for lg in self.loggers:
                    lg.log_eval(step, logs)
                self.save_best_checkpoint(logs, step, last_cs)
                continue
            samples, cs, pass_rate, t_gen = item
            t_total0 = t_wait
            status, global_step = self.train_step(samples, global_step)
            self.rollout_slots.put(global_step)
            status["timing/generation"] = t_gen
            status["timing/step_total"] = time.time() - t_total0      # wall clock including queue wait
            if a.algo.dynamic_filtering_enable:
                status["dynamic_filtering_pass_rate"] = pass_rate
            print(f"global step {global_step}: " + ", ".join(
                f"{k}={v:.4g}" for k, v in status.items() if isinstance(v, (int, float))), flush=True)
            last_cs = dict(cs, global_step=global_step)
            self.save_logs_and_checkpoints(global_step, status, last_cs)
        producer.join(timeout=60)
        for lg in self.loggers:
            lg.close()
        if self._errors:
            raise self._errors[0]
