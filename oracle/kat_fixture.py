"""Readers for the upstream known-answer test (test infrastructure).

The upstream project pins its whole inference chain with one script,
``unit_tests/models/unit_test_sorf.py`` (geometry, charges, expected energy and
forces as Python literals) plus a TorchScript archive
``unit_tests/models/saved_models/model_sorf.pt``.  ``tests/golden/upstream/``
holds a copy of the archive and the parsed literals, written by
``tests/golden/upstream/make_upstream_golden.py`` with the readers below.

* ``load_torchscript_tensors`` decodes the archive without registering any
  custom operator and without a GPU: the archive is a zip, ``data.pkl`` is a
  pickle whose persistent ids point at raw little-endian blobs.
* ``parse_unit_test`` extracts the literals of the script by walking its AST;
  nothing in the script is executed.
"""

from __future__ import annotations

import ast
import pickle
import zipfile
from collections import OrderedDict

import numpy as np
import torch

_STORAGE_DTYPES = {
    'FloatStorage': torch.float32,
    'DoubleStorage': torch.float64,
    'LongStorage': torch.int64,
    'IntStorage': torch.int32,
    'BoolStorage': torch.bool,
    'HalfStorage': torch.float16,
}


class _Obj:
    """Stand-in for a scripted module class: keeps the attribute dict."""

    def __init__(self, *args):
        self.__dict__['_state'] = {}

    def __setstate__(self, state):
        self.__dict__['_state'] = state


class _StorageTag:
    def __init__(self, name):
        self.dtype = _STORAGE_DTYPES[name]


def _rebuild_tensor_v2(storage, offset, size, stride, requires_grad=False, backward_hooks=None, metadata=None):
    flat = storage
    t = torch.as_strided(flat, tuple(size), tuple(stride), offset) if len(size) else flat[offset].clone()
    return t.clone()


class _Unpickler(pickle.Unpickler):
    def __init__(self, fh, zf, prefix):
        super().__init__(fh)
        self._zf = zf
        self._prefix = prefix

    def find_class(self, module, name):
        if module.startswith('__torch__'):
            return type(name, (_Obj,), {})
        if module == 'torch._utils' and name == '_rebuild_tensor_v2':
            return _rebuild_tensor_v2
        if module == 'torch' and name in _STORAGE_DTYPES:
            return _StorageTag(name)
        if module == 'torch' and name == 'device':
            return lambda *a: 'device:' + str(a[0])
        if module == 'collections' and name == 'OrderedDict':
            return OrderedDict
        raise pickle.UnpicklingError(f"unexpected global {module}.{name}")

    def persistent_load(self, pid):
        kind, tag, key, _device, numel = pid
        assert kind == 'storage'
        raw = self._zf.read(f'{self._prefix}/data/{key}')
        arr = np.frombuffer(raw, dtype=torch.empty(0, dtype=tag.dtype).numpy().dtype, count=numel)
        return torch.from_numpy(arr.copy())


def _flatten(obj, prefix, out):
    for k, v in obj._state.items():
        name = f'{prefix}{k}'
        if isinstance(v, _Obj):
            _flatten(v, name + '.', out)
        else:
            out[name] = v


def load_torchscript_tensors(path: str) -> dict:
    """Attribute dict (nested names joined with '.') of a saved TorchScript model."""
    with zipfile.ZipFile(path) as zf:
        pkl = [n for n in zf.namelist() if n.endswith('/data.pkl')][0]
        prefix = pkl.rsplit('/', 1)[0]
        import io
        root = _Unpickler(io.BytesIO(zf.read(pkl)), zf, prefix).load()
    out = {}
    _flatten(root, '', out)
    return out


def parse_unit_test(path: str) -> dict:
    """Literal assignments (``coordinates``, ``charges``, ``ref_energy``, ``ref_forces`` ...)."""
    with open(path) as fh:
        tree = ast.parse(fh.read())
    wanted = {'energy', 'coordinates', 'actual_forces', 'charges', 'ref_energy', 'ref_forces'}
    found = {}

    def literal(node):
        # np.array([...]) -> the list literal; plain numbers as they are; -x handled by literal_eval
        if isinstance(node, ast.Call) and getattr(node.func, 'attr', '') == 'array':
            return np.array(ast.literal_eval(node.args[0]))
        return ast.literal_eval(node)

    for node in ast.walk(tree):
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            name = node.targets[0].id
            if name in wanted and name not in found:
                try:
                    found[name] = literal(node.value)
                except (ValueError, SyntaxError):
                    pass
    return found
