"""Drop-in for the reference's ``heterofusedkernels`` package
(common/heterofusedkernels/__init__.py is empty; ``memory`` is its extension module)."""
