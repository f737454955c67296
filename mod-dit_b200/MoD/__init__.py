"""Drop-in `MoD` package: the `MoD.mod` modules keep the reference's names and signatures and run on the
sm_100a kernels of `moddit_b200`."""
