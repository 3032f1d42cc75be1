"""``paddle.version``"""
full_version = "3.0.0+b200"
major, minor, patch, rc = "3", "0", "0", "0"
istaged = True
commit = "unknown"
with_pip_cuda_libraries = "OFF"
cuda_version = "12.9"
cudnn_version = "unused"


def show():
    print(f"full_version: {full_version}\ncuda: {cuda_version}")


def cuda():
    return cuda_version


def cudnn():
    return cudnn_version


def nccl():
    import torch
    try:
        return ".".join(str(v) for v in torch.cuda.nccl.version())
    except Exception:  # noqa: BLE001
        return "0"
