"""Model tools and the built-in dataset catalogue over REST.

Parity: crates/axonml-server/src/api/tools.rs (inspect / convert / quantize / export of a stored
model version, the list of quantisation types) and api/builtin_datasets.rs (search, sources, one
entry, prepare).  Where the reference's convert / quantize handlers record a new file name and
sizes, these handlers really write the converted file next to the stored version and add it to the
model as a new version."""
from __future__ import annotations

import os

from .api import HttpError

_EXPORT_TARGETS = {
    "onnx": ("onnx", ["ONNX Runtime", "TensorRT", "OpenVINO"]),
    "safetensors": ("safetensors", ["HuggingFace Transformers", "PyTorch", "axonml"]),
    "json": ("json", ["any JSON reader"]),
    "axonml": ("axonml", ["axonml"]),
    "gguf": ("gguf", ["llama.cpp", "axonml serve --gguf"]),
}


def _human(nbytes: float) -> str:
    for unit in ("B", "KB", "MB", "GB"):
        if nbytes < 1024 or unit == "GB":
            return f"{nbytes:.2f} {unit}" if unit != "B" else f"{int(nbytes)} B"
        nbytes /= 1024
    return f"{nbytes:.2f} GB"


def register(app) -> None:
    r = app.router

    def _version(req) -> tuple:
        model = app.registry.get_model(req.params["id"])
        if model.get("user_id") not in (req.user_id, None) and req.claims.role != "admin":
            raise HttpError(403, "this item belongs to another user")
        return model, app.registry.get_version(req.params["id"], int(req.params["version"]))

    def _sibling(version: dict, ext: str, tag: str = "") -> str:
        stem = os.path.splitext(version["file_path"])[0]
        return f"{stem}{('.' + tag) if tag else ''}.{ext}"

    def _add_version(model: dict, path: str, note: dict) -> dict:
        with open(path, "rb") as f:
            data = f.read()
        os.remove(path)
        return app.registry.upload_version(model["id"], os.path.basename(path), data, note, None)

    # ------------------------------------------------------------------ inspect
    def inspect_model(req):
        from ...cli.workspace import model_summary
        model, v = _version(req)
        s = model_summary(v["file_path"])
        rows = s["entries"]
        layers = [{"index": i, "name": t["name"], "layer_type": _layer_type(t["name"], t["shape"]), "shape": t["shape"],
                   "num_params": t["numel"], "dtype": t["dtype"]} for i, t in enumerate(rows)]
        n = sum(t["numel"] for t in rows)
        return {"name": model["name"], "format": s["format"], "file_size": os.path.getsize(v["file_path"]),
                "num_parameters": n, "num_layers": len({t["name"].rsplit(".", 1)[0] for t in rows}), "layers": layers,
                "metadata": {"version": str(v["version"]), "file": os.path.basename(v["file_path"])},
                "memory_fp32": _human(4 * n), "memory_fp16": _human(2 * n),
                "trainable_params": sum(t["numel"] for t in rows if "running_" not in t["name"] and "num_batches" not in t["name"]),
                "non_trainable_params": sum(t["numel"] for t in rows if "running_" in t["name"] or "num_batches" in t["name"])}

    def _layer_type(name: str, shape) -> str:
        leaf = name.rsplit(".", 1)[-1]
        if "running_" in leaf or leaf == "num_batches_tracked":
            return "BatchNorm statistic"
        if len(shape) == 4:
            return "Conv2d"
        if len(shape) == 3:
            return "Conv1d"
        if len(shape) == 2:
            return "Embedding" if "embed" in name.lower() else "Linear"
        return "bias / norm" if len(shape) == 1 else "scalar"

    # ------------------------------------------------------------------ convert / export
    def _write_as(src: str, dst: str, fmt: str) -> int:
        """Writes the tensors of ``src`` to ``dst`` in ``fmt``; returns the parameter count."""
        from ...cli.commands import _state_of
        from ...serialize import save_state_dict
        sd, _ = _state_of(src)
        tensors = sd.to_tensors()
        if fmt == "onnx":
            from ...cli.commands import model_from_file
            from ...onnx import export_module, export_onnx
            module, _ = model_from_file(src)
            first = next(p for p in module.parameters() if p.dim() >= 2)
            if first.dim() != 2:
                raise HttpError(400, "ONNX export over REST covers models that start with a Linear layer; use `axonml export` with --input-shape for others")
            export_onnx(export_module(module, [1, int(first.shape[1])]), dst)
        elif fmt == "gguf":
            from ...quant.gguf import write_gguf
            write_gguf(dst, {k: v.float() for k, v in tensors.items()}, {"general.name": os.path.basename(src)})
        elif fmt in ("safetensors", "json", "axonml"):
            save_state_dict(sd, dst)
        else:
            raise HttpError(400, f"unknown target format {fmt!r} (one of {', '.join(sorted(_EXPORT_TARGETS))})")
        return sum(v.numel() for v in tensors.values())

    def convert_model(req):
        from ..app.registry import detect_format
        model, v = _version(req)
        (target,) = req.need("target_format")
        target = target.lower()
        if target not in _EXPORT_TARGETS:
            raise HttpError(400, f"unknown target format {target!r} (one of {', '.join(sorted(_EXPORT_TARGETS))})")
        dst = _sibling(v, _EXPORT_TARGETS[target][0], "converted")
        n = _write_as(v["file_path"], dst, target)
        size = os.path.getsize(dst)
        new = _add_version(model, dst, {"converted_from": v["version"], "format": target})
        warnings = ["optimisation passes apply to ONNX graphs only"] if req.json.get("optimize") and target != "onnx" else []
        return 201, {"input_file": os.path.basename(v["file_path"]), "output_file": os.path.basename(new["file_path"]),
                     "input_format": detect_format(v["file_path"]), "output_format": target,
                     "input_size": os.path.getsize(v["file_path"]), "output_size": size, "num_parameters": n,
                     "warnings": warnings, "version": new["version"]}

    def export_model(req):
        model, v = _version(req)
        (target,) = req.need("target")
        target = target.lower()
        if target == "torchscript":
            raise HttpError(400, "TorchScript export is not available: export to onnx or safetensors instead")
        if target not in _EXPORT_TARGETS:
            raise HttpError(400, f"unknown export target {target!r} (one of {', '.join(sorted(_EXPORT_TARGETS))})")
        dst = _sibling(v, _EXPORT_TARGETS[target][0], "export")
        _write_as(v["file_path"], dst, target)
        size = os.path.getsize(dst)
        new = _add_version(model, dst, {"exported_from": v["version"], "format": target})
        return 201, {"output_file": os.path.basename(new["file_path"]), "format": target, "size": size,
                     "compatible_with": _EXPORT_TARGETS[target][1], "version": new["version"]}

    # ------------------------------------------------------------------ quantize
    def quantize_model(req):
        from ...cli.commands import _state_of, quant_type
        from ...quant.gguf import write_gguf
        from ...quant.quantize import quantize_tensor
        model, v = _version(req)
        (target,) = req.need("target_type")
        try:
            qt = quant_type(target)
        except SystemExit as e:
            raise HttpError(400, str(e)) from None
        sd, _ = _state_of(v["file_path"])
        out, n, src_types = {}, 0, set()
        for k, t in sd.to_tensors().items():
            n += t.numel()
            src_types.add(str(t.dtype).replace("torch.", ""))
            if qt.is_block_quantized() and t.dim() >= 2 and t.shape[-1] % qt.block_size() == 0:
                out[k] = quantize_tensor(t.float(), qt)
            elif not qt.is_block_quantized() and t.is_floating_point():
                out[k] = quantize_tensor(t.float(), qt)
            else:
                out[k] = t.float()
        dst = _sibling(v, "gguf", qt.value)
        write_gguf(dst, out, {"general.name": model["name"], "general.quantization": qt.name})
        size, before = os.path.getsize(dst), os.path.getsize(v["file_path"])
        new = _add_version(model, dst, {"quantized_from": v["version"], "quant_type": qt.name})
        return 201, {"input_file": os.path.basename(v["file_path"]), "output_file": os.path.basename(new["file_path"]),
                     "source_type": "/".join(sorted(src_types)), "target_type": qt.name, "input_size": before,
                     "output_size": size, "compression_ratio": before / max(size, 1), "num_parameters": n,
                     "version": new["version"]}

    def quantization_types(req):
        from ...quant.types import QuantType
        notes = {"Q4_0": "4-bit blocks of 32, one scale", "Q4_1": "4-bit blocks of 32, scale and minimum",
                 "Q5_0": "5-bit blocks of 32, one scale", "Q5_1": "5-bit blocks of 32, scale and minimum",
                 "Q8_0": "8-bit blocks of 32, one scale", "Q4_K": "4-bit super-blocks of 256 with 6-bit sub-scales",
                 "F16": "half precision", "BF16": "bfloat16", "F32": "full precision"}
        return {"types": [{"name": q.name, "bits_per_weight": q.bits_per_value(), "description": notes[q.name]} for q in QuantType]}

    # ------------------------------------------------------------------ built-in datasets
    def search_builtin(req):
        from ...data.catalog import search_datasets
        return search_datasets(req.q("query", "") or req.q("q", ""), req.q("source", None), req.q("limit", 10, int))

    def dataset_sources(req):
        from ...data import catalog
        return catalog.SOURCES

    def builtin_info(req):
        from ...data.catalog import get_dataset_info
        d = get_dataset_info(req.params["id"])
        if d is None:
            raise HttpError(404, f"Dataset '{req.params['id']}' not found")
        return d

    def prepare_builtin(req):
        d = dict(builtin_info(req))
        d.setdefault("loading_code", f"# axonml dataset download {d['id']}\nfrom axonml_b200.{d['loader'].rsplit('.', 1)[0]} import {d['loader'].rsplit('.', 1)[1]}")
        return d

    r.add("GET", "/api/models/:id/versions/:version/inspect", inspect_model)
    r.add("POST", "/api/models/:id/versions/:version/convert", convert_model)
    r.add("POST", "/api/models/:id/versions/:version/quantize", quantize_model)
    r.add("POST", "/api/models/:id/versions/:version/export", export_model)
    r.add("GET", "/api/tools/quantization-types", quantization_types)
    r.add("GET", "/api/builtin-datasets/search", search_builtin)
    r.add("GET", "/api/builtin-datasets/sources", dataset_sources)
    r.add("GET", "/api/builtin-datasets/:id", builtin_info)
    r.add("POST", "/api/builtin-datasets/:id/prepare", prepare_builtin)
