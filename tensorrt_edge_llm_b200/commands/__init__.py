"""Argument-parsing front ends behind the ``trtedge`` sub-commands (``tensorrt_edgellm/scripts/*.py``)."""
