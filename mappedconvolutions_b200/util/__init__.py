from .point_functions import knn
from .spherical_projections import (convert_spherical_to_image, equirectangular_meshgrid,
                                    get_projection_map, reverse_gnomonic_projection_map)

__all__ = ["knn", "get_projection_map", "reverse_gnomonic_projection_map",
           "convert_spherical_to_image", "equirectangular_meshgrid"]
