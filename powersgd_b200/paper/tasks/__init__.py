"""Task factory (paper-code/tasks/__init__.py:1-20)."""


def build(task_name, seed, device, timer, **kwargs):
    if task_name == "Cifar":
        from .cifar import CifarTask

        extra = {k: kwargs[k] for k in ("train_size", "test_size") if k in kwargs}
        return CifarTask(seed=seed, device=device, timer=timer, architecture=kwargs.get("task_architecture", "ResNet18"), **extra)
    if task_name in ("LanguageModeling", "LSTM"):
        from .language_modeling import LanguageModelingTask

        extra = {k: kwargs[k] for k in ("vocab", "train_tokens", "valid_tokens", "hidden", "layers") if k in kwargs}
        return LanguageModelingTask(seed=seed, device=device, timer=timer, batch_size=kwargs.get("optimizer_batch_size"), **extra)
    raise ValueError("Unknown task name")
