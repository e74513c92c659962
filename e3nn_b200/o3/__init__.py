from ._irreps import Irrep, Irreps
from ._linear import Linear
from ._norm import Norm
from ._rotation import angles_to_matrix, matrix_to_angles, rand_angles, rand_matrix
from ._spec import Instruction
from ._spherical_harmonics import SphericalHarmonics, spherical_harmonics
from ._tensor_product import ElementwiseTensorProduct, FullTensorProduct, FullyConnectedTensorProduct, TensorProduct, TensorSquare
from ._tp_linear import TensorProductLinear
from ._wigner import wigner_3j, wigner_D

__all__ = [
    "Irrep", "Irreps", "Linear", "Norm", "Instruction", "SphericalHarmonics", "spherical_harmonics",
    "ElementwiseTensorProduct", "FullTensorProduct", "FullyConnectedTensorProduct", "TensorProduct", "TensorProductLinear", "TensorSquare", "wigner_3j", "wigner_D",
    "rand_matrix", "rand_angles", "angles_to_matrix", "matrix_to_angles",
]
