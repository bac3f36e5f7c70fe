from .modules import NeighborhoodAttention1D, NeighborhoodAttention2D, NeighborhoodAttention3D

__all__ = ["NeighborhoodAttention1D", "NeighborhoodAttention2D", "NeighborhoodAttention3D"]
