from . import icosphere
from .icosphere import (generate_icosphere, image_to_sphere_resample_map, one_ring, pooling_map,
                        vertex_kernel_map)
from .point_functions import knn
from .spherical_projections import (convert_spherical_to_image, equirectangular_meshgrid,
                                    get_projection_map, reverse_gnomonic_projection_map)

__all__ = ["knn", "get_projection_map", "reverse_gnomonic_projection_map",
           "convert_spherical_to_image", "equirectangular_meshgrid", "icosphere",
           "generate_icosphere", "one_ring", "vertex_kernel_map", "pooling_map",
           "image_to_sphere_resample_map"]
