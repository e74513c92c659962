from ._fc import FullyConnectedNet, bessel, normalize2mom_constant
from ._interaction import InteractionBlock, radius_graph_pbc

__all__ = ["FullyConnectedNet", "bessel", "normalize2mom_constant", "InteractionBlock", "radius_graph_pbc"]
