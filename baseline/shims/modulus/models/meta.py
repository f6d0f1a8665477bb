from dataclasses import dataclass


@dataclass
class ModelMetaData:
    name: str = "ModulusModule"
    jit: bool = False
    cuda_graphs: bool = False
    amp: bool = False
    amp_cpu: bool = None
    amp_gpu: bool = None
    torch_fx: bool = False
    bf16: bool = False
    onnx: bool = False
    onnx_gpu: bool = None
    onnx_cpu: bool = None
    onnx_runtime: bool = False
    trt: bool = False
    var_dim: int = -1
    func_torch: bool = False
    auto_grad: bool = False
