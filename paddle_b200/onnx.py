"""``paddle.onnx.export`` (python/paddle/onnx/export.py) delegates to the external paddle2onnx package in the
reference; no ONNX exporter is bundled here."""


def export(layer, path, input_spec=None, opset_version=9, **configs):
    raise NotImplementedError("ONNX export needs the external paddle2onnx converter, which is not part of this build; "
                              "use paddle.jit.save for deployment through paddle.inference")
