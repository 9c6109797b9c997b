"""SparseConvNetTensor: features + the Metadata that says where they live
(reference: sparseconvnet/sparseConvNetTensor.py:13-66)."""


class SparseConvNetTensor(object):
    def __init__(self, features=None, metadata=None, spatial_size=None, recompute_all=False, new_points=None):
        self.features = features
        self.metadata = metadata
        self.spatial_size = spatial_size
        # set by InputLayer in the exact incremental mode: the tensor holds the whole merged scene, so the
        # layers downstream run their full-frame path; new_points = (first, count) of the frame's own points
        self.recompute_all = recompute_all
        self.new_points = new_points
        # (BatchNormalization module, its result on these features) when the convolution that made the features
        # also formed that module's output in its epilogue; not carried over by like()
        self.bn_ready = None

    def get_spatial_locations(self, spatial_size=None):
        """LongTensor [nActive, 4]: x, y, z, batch index of every active site, in row order."""
        return self.metadata.getSpatialLocations(self.spatial_size if spatial_size is None else spatial_size)

    def like(self, features, spatial_size=None):
        """A tensor on the same metadata carrying other features."""
        return SparseConvNetTensor(features, self.metadata, self.spatial_size if spatial_size is None else spatial_size,
                                   self.recompute_all, self.new_points)

    def detach(self):
        return self.like(self.features.detach())

    def to(self, device):
        self.features = self.features.to(device)
        return self

    def cuda(self):
        self.features = self.features.cuda()
        return self

    def cpu(self):
        self.features = self.features.cpu()
        return self

    def type(self, t=None):
        if t:
            self.features = self.features.type(t)
            return self
        return self.features.type()

    def __repr__(self):
        return "SparseConvNetTensor<<features.shape=%r, spatial size=%r>>" % (
            None if self.features is None else tuple(self.features.shape), self.spatial_size)
