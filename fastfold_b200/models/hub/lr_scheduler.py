"""Learning-rate schedule of supplement 1.11.3: linear warm-up, plateau, then stepwise exponential decay.

``AlphaFoldLRScheduler(optimizer, last_epoch=-1, base_lr=0, max_lr=1e-3, warmup_no_steps=1000, start_decay_after_n_steps=50000,
decay_every_n_steps=50000, decay_factor=0.95)``; same contract as fastfold/model/hub/lr_scheduler.py:28-97.  Works with any
object that has ``param_groups`` (a ``torch.optim`` optimizer) or an ``lr`` attribute (``FlatAdamTrainer``).
"""


class AlphaFoldLRScheduler:
    def __init__(self, optimizer, last_epoch=-1, verbose=False, base_lr=0.0, max_lr=0.001, warmup_no_steps=1000,
                 start_decay_after_n_steps=50000, decay_every_n_steps=50000, decay_factor=0.95):
        if warmup_no_steps > start_decay_after_n_steps:
            raise ValueError("warmup_no_steps must not exceed start_decay_after_n_steps")
        self.optimizer = optimizer
        self.last_epoch = last_epoch
        self.base_lr, self.max_lr = base_lr, max_lr
        self.warmup_no_steps = warmup_no_steps
        self.start_decay_after_n_steps = start_decay_after_n_steps
        self.decay_every_n_steps = decay_every_n_steps
        self.decay_factor = decay_factor
        self.step()

    def lr_at(self, step_no):
        if step_no <= self.warmup_no_steps:
            return self.base_lr + (step_no / max(1, self.warmup_no_steps)) * self.max_lr
        if step_no > self.start_decay_after_n_steps:
            steps_since_decay = step_no - self.start_decay_after_n_steps
            exp = (steps_since_decay // self.decay_every_n_steps) + 1
            return self.max_lr * (self.decay_factor ** exp)
        return self.max_lr

    def get_lr(self):
        return [self.lr_at(self.last_epoch)]

    def step(self):
        self.last_epoch += 1
        lr = self.lr_at(self.last_epoch)
        if hasattr(self.optimizer, "param_groups"):
            for g in self.optimizer.param_groups:
                g["lr"] = lr
        else:
            self.optimizer.lr = lr
        return lr

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, state_dict):
        self.__dict__.update(state_dict)
