"""The research training loop end to end on CPU with tiny synthetic tasks."""
import os

import pytest
import torch

from powersgd_b200.paper import train


@pytest.fixture
def small_config(tmp_path):
    saved = dict(train.config)
    saved_out = train.output_dir
    train.output_dir = str(tmp_path)
    train.config.update(num_epochs=1, optimizer_batch_size=16, max_batches_per_epoch=4, log_verbosity=0, device="cpu",
                        task_architecture="LeNet", train_size=256, test_size=64, distributed_backend="gloo",
                        optimizer_scale_lr_with_warmup_epochs=0, optimizer_learning_rate=0.01, optimizer_conv_learning_rate=0.01)
    yield train.config
    train.config.clear()
    train.config.update(saved)
    train.output_dir = saved_out


@pytest.mark.parametrize("reducer,extra", [("ExactReducer", {}), ("RankKReducer", {"optimizer_reducer_rank": 2}),
                                           ("TopKReducer", {"optimizer_reducer_compression": 0.1}),
                                           ("SignAndNormReducer", {})])
def test_train_loop_runs(small_config, reducer, extra):
    small_config.update(optimizer_reducer=reducer, **extra)
    task, red, bits = train.main()
    assert all(torch.isfinite(p).all() for p in task.state)
    assert os.path.exists(os.path.join(train.output_dir, "timer_summary.json"))
    assert bits >= 0


def test_language_model_task_and_checkpoint_resume(small_config, tmp_path):
    small_config.update(task="LanguageModeling", optimizer_reducer="RankKReducer", optimizer_reducer_rank=2, vocab=200,
                        train_tokens=4000, valid_tokens=1000, hidden=16, layers=1, optimizer_batch_size=4, checkpoints=[0])
    task, red, bits = train.main()
    path = os.path.join(train.output_dir, "epoch_000")
    assert os.path.exists(path)
    small_config.update(resume_from=path, num_epochs=2, checkpoints=[])
    task2, red2, bits2 = train.main()
    assert bits2 > bits
    assert red2.p_memory is not None


def test_learning_rate_schedule(small_config):
    small_config.update(optimizer_scale_lr_with_warmup_epochs=5, optimizer_scale_lr_with_factor=4.0,
                        optimizer_learning_rate=0.1, optimizer_decay_at_epochs=[10, 20], optimizer_decay_with_factor=10.0)
    assert train.get_learning_rate(0.0, "linear.weight") == pytest.approx(0.1)
    assert train.get_learning_rate(2.5, "linear.weight") == pytest.approx(0.25)
    assert train.get_learning_rate(7.0, "linear.weight") == pytest.approx(0.4)
    assert train.get_learning_rate(12.0, "linear.weight") == pytest.approx(0.04)
    assert train.get_learning_rate(25.0, "linear.weight") == pytest.approx(0.004)
    assert train.is_conv_param("layer1.0.conv1.weight") and not train.is_conv_param("linear.weight")
    assert train.is_batchnorm_param("layer1.0.bn1.weight") and not train.is_batchnorm_param("bn.weight")
    assert train.get_weight_decay(0, "layer1.0.bn1.bias") == 0.0
