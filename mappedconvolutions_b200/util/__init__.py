from .point_functions import knn

__all__ = ["knn"]
