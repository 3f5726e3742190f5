"""GPU-derived configuration helpers (python/yirage/utils.py)."""
import torch


def get_shared_memory_capacity(target_cc):
    caps = {70: 96, 75: 64, 80: 163, 86: 99, 89: 99, 90: 223, 100: 227}
    if target_cc not in caps:
        raise AssertionError("Unsupported compute capacity: {}".format(target_cc))
    return caps[target_cc] * 1024


def get_scheduler(sm_cnt, worker):
    scheduler = 4 * (sm_cnt - worker)
    assert scheduler > 0, "worker count is not compatible with sm count on the GPU"
    return scheduler


def get_configurations_from_gpu(rank):
    """(num_workers, num_schedulers) as the reference derives them from the SM count
    (python/yirage/utils.py:39-57).  The values keep the shapes callers size with them
    (argmax partial buffers are [tokens, num_workers]); the B200 runtime itself has no
    scheduler CTAs and runs a worker on every SM regardless."""
    props = torch.cuda.get_device_properties(rank)
    sm_cnt = props.multi_processor_count
    print("sm_cnt: ", sm_cnt)
    if sm_cnt >= 160:
        worker = 144
    elif sm_cnt >= 132:
        worker = 128
    elif sm_cnt >= 108:
        worker = 96
    elif sm_cnt >= 68:
        worker = 64
    elif sm_cnt >= 40:
        worker = 30
    else:
        worker = 20
    return worker, get_scheduler(sm_cnt, worker)
