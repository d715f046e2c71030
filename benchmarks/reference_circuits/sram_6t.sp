* six-transistor SRAM cell: write a 0 then a 1 through the access transistors
VDD vdd 0 DC 1.8
VWL wl 0 PULSE(0 1.8 200p 20p 20p 300p 1n)
VBL bl 0 PULSE(0 1.8 900p 20p 20p 900p 2n)
VBLB blb 0 PULSE(1.8 0 900p 20p 20p 900p 2n)
* cross-coupled inverters
MP1 q qb vdd vdd pch w=0.6u l=180n
MN1 q qb 0 0 nch w=1.2u l=180n
MP2 qb q vdd vdd pch w=0.6u l=180n
MN2 qb q 0 0 nch w=1.2u l=180n
* access transistors
MA1 bl wl q 0 nch w=0.8u l=180n
MA2 blb wl qb 0 nch w=0.8u l=180n
CQ q 0 1f
CQB qb 0 1f
.ic v(q)=1.8 v(qb)=0
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.tran 1p 2n
.end
