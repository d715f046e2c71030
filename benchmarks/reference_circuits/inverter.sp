* CMOS inverter driven by a pulse, 10 fF load
VDD vdd 0 DC 1.8
VSS vss 0 DC 0
VIN in 0 PULSE(0 1.8 100p 20p 20p 400p 1n)
MP out in vdd vdd pch w=2u l=180n
MN out in vss vss nch w=1u l=180n
CL out 0 10f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
.tran 1p 2n
.end
