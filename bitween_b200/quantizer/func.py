def _set_module(model, submodule_key, module):
    """Replace the submodule at the dotted path `submodule_key` (e.g. "layers.0.fc1") of `model`
    by `module` (same helper as bitween/quantizer/func.py:1-15)."""
    *parents, leaf = submodule_key.split(".")
    cur = model
    for name in parents:
        cur = getattr(cur, name)
    setattr(cur, leaf, module)
