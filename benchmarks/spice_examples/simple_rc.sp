* RC low-pass fed from the supply; n1 charges towards vdd_val with tau = 1 k * 1 f = 1 ps
.param vdd_val=1.8
VDD vdd 0 DC vdd_val
R1 vdd n1 1k
C1 n1 0 1f
.ic v(n1)=0
.tran 1p 10p
.end
