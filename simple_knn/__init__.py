"""Import-path stand-in for the reference's simple-knn submodule: ``from simple_knn._C import distCUDA2``
(classes/point_cloud.py:10) resolves to the implementation in librgx.so."""
