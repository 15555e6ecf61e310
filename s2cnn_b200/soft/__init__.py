from .s2_conv import S2Convolution
from .so3_conv import SO3Convolution, SO3Shortcut
from .so3_integrate import so3_integrate, so3_relu_integrate
from .so3_rotation import so3_rotation
