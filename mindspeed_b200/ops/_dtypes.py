import torch

CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def code(dtype) -> int:
    try:
        return CODE[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported by the sm_100a kernels") from None
